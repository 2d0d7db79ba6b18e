// Linear layer with the op that follows it folded into the GEMM epilogue (sm_100a: tcgen05 + TMEM + TMA).
//
// The reference runs every projection as a library GEMM that writes a bf16 matrix, then add_bias_bf16 as
// a read-modify-write of that matrix (src/core/weights.cpp:159-177, `linear_one`), and for the attention
// out-projection and the second MLP projection a gated_residual that reads it once more
// (src/models/qwen_image/dit.cpp:304-305, 313-314; src/models/minimax_h3/dit.cpp:238, 245).  Here the GEMM
// keeps its accumulator in tensor memory and the epilogue applies, per element and in the reference's
// order and roundings,
//     y  = bf16(acc)                       what the library GEMM would have stored
//     y  = bf16(y + bias[col])             add_bias_bf16 (src/kernels/ops.cu:249-262), when a bias is given
//     x += act(gate[col]) * y              gated_residual (src/kernels/ops.cu:73-84), EPI_RESIDUAL
// so the bf16 projection output never exists in memory: 2·M·N bytes written and 4·M·N (bias) + 2·M·N
// (residual) bytes re-read disappear.  EPI_STORE writes y as bf16 instead (a plain linear layer), optionally through
// GELU (the reference's linear -> gelu_tanh_inplace, src/models/qwen_image/dit.cpp:192-193).  EPI_SWIGLU is the first
// MLP projection with silu_mul in its epilogue (linear(gate_up) -> silu_mul, src/models/qwen_image/dit.cpp:309-312,
// src/models/minimax_h3/dit.cpp:241-242): a tile's 256 accumulator columns are 128 gate columns and the 128 up
// columns F further along the weight's rows, the epilogue writes silu(gate) * up, and the [M, 2F] projection
// (written once, read once) never exists.
//
// y = A[M, K] · W[N, K]^T, both operands bf16 and K-major (activations row-major, weights in the
// [out, in] layout the reference keeps them in), fp32 accumulation.
//
// Kernel shape: one persistent CTA per SM, 320 threads.
//   warp 0, one lane:  TMA producer - 128 x 64 tiles of A and 256 x 64 tiles of W (128-byte swizzle) into a
//                      4-stage shared-memory ring, completing on `full` mbarriers;
//   warp 1, one lane:  issues tcgen05.mma (M 128, N 256, K 16, cta_group::1) from shared-memory descriptors
//                      into one of two 256-column TMEM accumulators; tcgen05.commit releases a stage
//                      (`empty`) and publishes a finished accumulator (`acc_full`);
//   warps 2-9:         epilogue - each thread owns one row of the tile (its TMEM lane; the warp's index modulo 4
//                      selects the lane quarter) and one half of its 256 columns (warps 2-5 the first, 6-9 the
//                      second), reads the accumulator 32 columns at a time (tcgen05.ld 32x32b), applies the chain
//                      above and updates x with 128-bit accesses; the other accumulator is being filled meanwhile.
// Every mbarrier wait is bounded (bulk_copy.cuh); on a timeout the role records kErrBulkTimeout in the
// device error word and leaves its loop, the CTA still meets at the final barrier and frees its TMEM.
// Every copy lands in the shared memory of the CTA that issued it (no copy is broadcast to several CTAs), so the
// file may travel to multi-GPU runs.
#include <cuda.h>

#include <atomic>

#include "act_math.cuh"
#include "bulk_copy.cuh"
#include "common.cuh"
#include "tuning.h"

namespace mxk {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int kStageA = BM * BK * 2;  // 16 KB: this CTA's 128 rows of A
// CTAS = 1: the CTA holds the whole 256-row W tile (32 KB), 4 stages.  CTAS = 2 (a pair of CTAs in a cluster working
// on a 256 x 256 tile, tcgen05 cta_group::2): each CTA holds its 128 rows of A and HALF of the W tile (16 KB), 6 stages.
template <int CTAS> constexpr int kStageB = BN / CTAS * BK * 2;
template <int CTAS> constexpr int kStages = CTAS == 1 ? 4 : 6;
constexpr int kAccCols = BN;                                  // fp32 columns of one accumulator
constexpr int kTmemCols = 2 * kAccCols;                       // two accumulators: all 512 columns
constexpr int kEpiWarps = 8, kEpiThreads = 32 * kEpiWarps;
constexpr int kThreads = 64 + kEpiThreads;  // producer warp, MMA warp, epilogue warps
constexpr int EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_QKV = 2, EPI_SWIGLU = 3;
// output columns one tile covers: EPI_SWIGLU spends half of the accumulator on the up half of the projection
template <int EPI> constexpr int kTileCols = EPI == EPI_SWIGLU ? BN / 2 : BN;
constexpr int kTurnRow = 80;   // bytes between rows of the residual epilogue's transposition tile
constexpr int kHeadDim = 128;  // EPI_QKV: a 256-column tile is exactly two heads, one per half of the epilogue warps

struct LinearArgs {
  int64_t M, N, K;
  const float* bias;  // fp32 [N] or null
  bf16* y;            // EPI_STORE, EPI_SWIGLU: bf16 [M, N]
  int act;            // EPI_STORE: 0 none, 1 GELU (tanh form), 2 GELU (erf form) applied to the stored value
  float* x;           // EPI_RESIDUAL: fp32 [M, N], updated in place
  MxkRowMod gate;     // EPI_RESIDUAL
  int gate_tanh;
  // EPI_QKV: the N = n_tensors * H * 128 output columns are n_tensors projections of H heads each; head h of
  // tensor i is normalised with norm_w[i] (null: no norm), rotated (rot[i], mode[i]) and stored to out[i] [M, H, 128]
  int H;
  const float* norm_w[3];
  bf16* out[3];
  int rot[3], mode[3];
  float eps;
  const float* cos;
  const float* sin;
  int group_m;  // tile order: bands of this many row tiles, walked down the rows first (see tile_coords)
  int* err;
};

// Tile t of the persistent loop -> (row tile, column tile).  Tiles are numbered band by band; a band is `group_m` row
// tiles high and as wide as the matrix, and inside a band the number runs down the rows first.  The CTAs of one wave
// (consecutive numbers) then cover a block of about group_m x (CTAs / group_m) tiles: per wave they read group_m row
// tiles of A and CTAs / group_m column tiles of W instead of one or two row tiles and ALL of W, which matters once W
// is larger than L2 (a QKV projection of 15360 x 5120 is 157 MB).
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& mt, int& nt) {
  const int band = t / (group_m * tiles_n), first = band * group_m;
  const int rows = tiles_m - first < group_m ? tiles_m - first : group_m;  // the last band may be lower
  const int r = t - band * group_m * tiles_n;
  mt = first + r % rows, nt = r / rows;
}

template <int CTAS>
struct __align__(1024) LinearSmem {
  unsigned char a[kStages<CTAS>][kStageA];
  unsigned char b[kStages<CTAS>][kStageB<CTAS>];
  float bias[BN];           // the tile's bias slice (0 when absent)
  float gate[2][BN];        // act(gate) for prefix rows [0] and target rows [1] (1 when absent); EPI_QKV: [0][0..127] = norm weights
  // EPI_RESIDUAL: per epilogue warp a 32 x 32 tile of bf16 y values, rows 80 bytes apart (64 of data: the padding keeps
  // both the row-per-lane writes and the four-rows-per-instruction reads off each other's banks)
  unsigned char turn[kEpiWarps][32 * kTurnRow];
  unsigned long long full[kStages<CTAS>], empty[kStages<CTAS>], acc_full[2], acc_empty[2], done;
  unsigned tmem_base;
};

__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
               "l"(map), "r"(bar), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_local(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// ---- helpers of the two-CTA form -----------------------------------------------------------------------
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address, in the cluster's shared window, of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ unsigned map_to_cta(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A pair's copy: lands in this CTA's shared memory, counts on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
// Arrives, once the MMAs issued so far have retired, on the barrier at this shared-memory offset in BOTH CTAs of the
// pair (the commit's own multicast form; it signals barriers and moves no data).
__device__ __forceinline__ void tc_commit_pair(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(static_cast<unsigned short>(3))
               : "memory");
}
// D[tmem of both CTAs] (+)= A[256 rows: 128 per CTA] * B[256 columns: 128 per CTA], issued by the pair's first CTA
__device__ __forceinline__ void tc_mma_pair(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// AND of a predicate over the epilogue threads (named barrier 1).
__device__ __forceinline__ bool epilogue_all(bool v) {
  unsigned r;
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\tbarrier.cta.red.and.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(r)
               : "r"(unsigned(v)), "n"(kEpiThreads)
               : "memory");
  return r != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
      "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tc_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// EPI_QKV: normalise, rotate and store one head (128 channels) of one token from its packed bf16 pairs.
// HC > 0: half mode, pairs (i, i + 16 HC) over the first 32 HC channels; HC == 0: interleaved pairs (2i, 2i + 1)
// over the first `rot` channels (a multiple of 16; 0: no rotation).  cos / sin rows are read with 128-bit
// non-coherent loads (the launcher checks their alignment), which the compiler may move ahead of the stores.
// Channels [C, C + 16) of a head from its packed bf16 pairs, normalised when a weight is given.
template <int C>
__device__ __forceinline__ void qkv_chunk(const unsigned (&P)[kHeadDim / 2], bool has_norm, float rstd, const float* nw, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const unsigned p = P[C / 2 + i];
    v[2 * i] = __uint_as_float(p << 16), v[2 * i + 1] = __uint_as_float(p & 0xffff0000u);
  }
  if (has_norm) {
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = v[i] * rstd * nw[C + i];
  }
}
template <int N4>
__device__ __forceinline__ void qkv_table(const float* p, float (&o)[4 * N4]) {  // N4 128-bit loads
#pragma unroll
  for (int j = 0; j < N4; j++) {
    const float4 q = __ldg(reinterpret_cast<const float4*>(p) + j);
    o[4 * j] = q.x, o[4 * j + 1] = q.y, o[4 * j + 2] = q.z, o[4 * j + 3] = q.w;
  }
}
__device__ __forceinline__ void qkv_store16(bf16* dst, const float (&o)[16]) {
  float lo[8], hi[8];
#pragma unroll
  for (int i = 0; i < 8; i++) lo[i] = o[i], hi[i] = o[8 + i];
  reinterpret_cast<uint4*>(dst)[0] = pack8(lo);
  reinterpret_cast<uint4*>(dst)[1] = pack8(hi);
}
// Half mode, chunk C of the first half: pairs (C + i, 16 HC + C + i); recursion over the chunks keeps every register
// index a constant.
template <int HC, int C>
__device__ __forceinline__ void qkv_half_chunks(const unsigned (&P)[kHeadDim / 2], bool has_norm, float rstd, const float* nw,
                                                const float* cr, const float* sr, bf16* orow) {
  if constexpr (C < 16 * HC) {
    constexpr int half = 16 * HC;
    float cs[16], sn[16], va[16], vb[16];
    qkv_table<4>(cr + C, cs);
    qkv_table<4>(sr + C, sn);
    qkv_chunk<C>(P, has_norm, rstd, nw, va);
    qkv_chunk<half + C>(P, has_norm, rstd, nw, vb);
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const float x0 = va[i], x1 = vb[i];
      va[i] = x0 * cs[i] - x1 * sn[i];
      vb[i] = fmaf(x0, sn[i], x1 * cs[i]);
    }
    qkv_store16(orow + C, va);
    qkv_store16(orow + half + C, vb);
    qkv_half_chunks<HC, C + 16>(P, has_norm, rstd, nw, cr, sr, orow);
  }
}
// Channels [C, 128) without rotation.
template <int C>
__device__ __forceinline__ void qkv_plain_chunks(const unsigned (&P)[kHeadDim / 2], bool has_norm, float rstd, const float* nw, bf16* orow) {
  if constexpr (C < kHeadDim) {
    float v[16];
    qkv_chunk<C>(P, has_norm, rstd, nw, v);
    qkv_store16(orow + C, v);
    qkv_plain_chunks<C + 16>(P, has_norm, rstd, nw, orow);
  }
}
// Interleaved mode (or none): pairs (2i, 2i + 1) over the first `rot` channels.
template <int C>
__device__ __forceinline__ void qkv_interleaved_chunks(const unsigned (&P)[kHeadDim / 2], bool has_norm, float rstd, const float* nw,
                                                       const float* cr, const float* sr, int rot, bf16* orow) {
  if constexpr (C < kHeadDim) {
    float v[16];
    if (C < rot) {
      float cs[8], sn[8];
      qkv_table<2>(cr + C / 2, cs);
      qkv_table<2>(sr + C / 2, sn);
      qkv_chunk<C>(P, has_norm, rstd, nw, v);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float x0 = v[2 * i], x1 = v[2 * i + 1];
        v[2 * i] = x0 * cs[i] - x1 * sn[i];
        v[2 * i + 1] = fmaf(x0, sn[i], x1 * cs[i]);
      }
    } else {
      qkv_chunk<C>(P, has_norm, rstd, nw, v);
    }
    qkv_store16(orow + C, v);
    qkv_interleaved_chunks<C + 16>(P, has_norm, rstd, nw, cr, sr, rot, orow);
  }
}
template <int HC>
__device__ __forceinline__ void qkv_head_store(const unsigned (&P)[kHeadDim / 2], bool has_norm, float rstd, const float* nw,
                                               const float* cr, const float* sr, int rot, bf16* orow) {
  if constexpr (HC > 0) {
    qkv_half_chunks<HC, 0>(P, has_norm, rstd, nw, cr, sr, orow);
    qkv_plain_chunks<32 * HC>(P, has_norm, rstd, nw, orow);
  } else {
    qkv_interleaved_chunks<0>(P, has_norm, rstd, nw, cr, sr, rot, orow);
  }
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) wide under the
// 128-byte swizzle: start address >> 4 in bits [0, 14); leading byte offset (unused by swizzled K-major
// layouts) 1 in [16, 30); stride byte offset = 1024 (eight rows) >> 4 in [32, 46); descriptor version 1 in
// [46, 48); layout type 2 (SWIZZLE_128B) in [61, 64).  The tile's base is 1024-byte aligned (base offset 0).
__device__ __forceinline__ uint64_t smem_desc_sw128(unsigned addr) {
  return uint64_t((addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}
// Instruction descriptor of kind::f16: fp32 accumulator (bits [4, 6) = 1), A and B bf16 ([7, 10) = [10, 13) = 1),
// both K-major (bits 15, 16 = 0), N >> 3 in [17, 23), M >> 4 in [24, 29).
template <int CTAS>
constexpr unsigned kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | (unsigned(BN >> 3) << 17) | (unsigned(BM * CTAS >> 4) << 24);

// CTAS = 2: launched as clusters of two CTAs along M.  The pair works on a 256 x 256 tile; CTA r of the pair owns rows
// [128 r, 128 r + 128) (its own TMEM lanes, its own epilogue) and loads those rows of A plus rows [128 r, 128 r + 128)
// of the W tile.  The first CTA's MMA thread issues cta_group::2 MMAs that read both CTAs' shared memory and write both
// CTAs' tensor memory.  Barriers: `full` lives in the first CTA and counts the bytes of both CTAs' copies; `empty` and
// `acc_full` exist in both CTAs and are signalled in both by the issuing thread's commits; `acc_empty`
// lives in the first CTA and collects the sixteen epilogue warps of the pair; `done` is the hand-shake before the
// tensor memory is freed and a CTA leaves (nobody may still signal into a CTA that has exited).
template <int EPI, int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
    linear_epilogue_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const LinearArgs a) {
  extern __shared__ unsigned char smem_raw[];
  // dynamic shared memory is 16-byte aligned by contract; the tiles need 1024 (the same offset in both CTAs of a pair)
  using Smem = LinearSmem<CTAS>;
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kSt = kStages<CTAS>;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned rank = CTAS == 2 ? cluster_rank() : 0u;
  constexpr int TN = kTileCols<EPI>;  // output columns per tile
  const int tiles_n = int((a.N + TN - 1) / TN), tiles_m = int((a.M + BM * CTAS - 1) / (BM * CTAS));
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = int((a.K + BK - 1) / BK);
  const int tile0 = int(blockIdx.x) / CTAS, tile_step = int(gridDim.x) / CTAS;

  if (tid == 0) {
    for (int i = 0; i < kSt; i++) mbar_init(smem_u32(&sm.full[i]), 1), mbar_init(smem_u32(&sm.empty[i]), 1);
    for (int i = 0; i < 2; i++) mbar_init(smem_u32(&sm.acc_full[i]), 1), mbar_init(smem_u32(&sm.acc_empty[i]), kEpiWarps * CTAS);
    mbar_init(smem_u32(&sm.done), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // one warp (the same one in both CTAs of a pair) allocates and later frees the tensor memory
    if (CTAS == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();  // both CTAs' barriers exist before either signals into the other
  tc_fence_after();
  const unsigned tmem_base = sm.tmem_base;
  pdl_wait();  // nothing above touches global memory

  bool ok = true;
  long issued = 0;  // producer: stage fills issued so far
  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer ----
      int st = 0;
      unsigned ph = 0;
      for (int t = tile0; t < n_tiles && ok; t += tile_step) {
        int mt, nt;
        tile_coords(t, tiles_m, tiles_n, a.group_m, mt, nt);
        // W rows of this CTA's part of the B tile.  EPI_SWIGLU: gate rows [nt TN, +128) then up rows [N + nt TN, +128);
        // in a pair the first CTA loads the gate rows and the second the up rows
        const int m0 = mt * BM * CTAS + int(rank) * BM;
        const int n0 = EPI == EPI_SWIGLU ? nt * TN + int(rank) * int(a.N) : nt * BN + int(rank) * (BN / CTAS);
        for (int kb = 0; kb < k_blocks; kb++, issued++) {
          if (issued >= kSt && !mbar_wait(smem_u32(&sm.empty[st]), ph ^ 1u)) {
            ok = false;
            break;
          }
          if (CTAS == 1) {
            const unsigned bar = smem_u32(&sm.full[st]);
            mbar_expect_tx(bar, kStageA + kStageB<1>);
            tma_load_2d(smem_u32(sm.a[st]), &map_a, kb * BK, m0, bar);
            if (EPI == EPI_SWIGLU) {  // two boxes of 128 rows: stacked they are the 256-row tile (16 KB = 16 swizzle groups each)
              tma_load_2d(smem_u32(sm.b[st]), &map_w, kb * BK, n0, bar);
              tma_load_2d(smem_u32(sm.b[st]) + kStageB<1> / 2, &map_w, kb * BK, n0 + int(a.N), bar);
            } else {
              tma_load_2d(smem_u32(sm.b[st]), &map_w, kb * BK, n0, bar);
            }
          } else {
            // the pair's `full` barrier is the first CTA's: it expects both CTAs' bytes, both CTAs' copies count on it
            if (rank == 0) mbar_expect_tx(smem_u32(&sm.full[st]), 2 * (kStageA + kStageB<2>));
            const unsigned bar = map_to_cta(smem_u32(&sm.full[st]), 0);
            tma_load_2d_pair(smem_u32(sm.a[st]), &map_a, kb * BK, m0, bar);
            tma_load_2d_pair(smem_u32(sm.b[st]), &map_w, kb * BK, n0, bar);
          }
          if (++st == kSt) st = 0, ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---- MMA issuer (the pair's first CTA only) ----
      int st = 0;
      unsigned ph = 0;
      int local = 0;
      for (int t = tile0; t < n_tiles && ok; t += tile_step, local++) {
        const int buf = local & 1;
        // the epilogue must have drained this accumulator (its previous use was two tiles ago)
        if (local >= 2 && !mbar_wait(smem_u32(&sm.acc_empty[buf]), unsigned(((local >> 1) - 1) & 1))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const unsigned tmem_d = tmem_base + unsigned(buf * kAccCols);
        for (int kb = 0; kb < k_blocks; kb++) {
          if (!mbar_wait(smem_u32(&sm.full[st]), ph)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = smem_desc_sw128(smem_u32(sm.a[st])), db = smem_desc_sw128(smem_u32(sm.b[st]));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {  // 32 bytes further along K per step: +2 in the (address >> 4) field
            if (CTAS == 1) tc_mma(tmem_d, da + uint64_t(2 * k), db + uint64_t(2 * k), kInstrDesc<1>, (kb | k) != 0 ? 1u : 0u);
            else tc_mma_pair(tmem_d, da + uint64_t(2 * k), db + uint64_t(2 * k), kInstrDesc<2>, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free once these MMAs have read it (in both CTAs of a pair)
          if (CTAS == 1) {
            tc_commit(smem_u32(&sm.empty[st]));
          } else {
            tc_commit_pair(smem_u32(&sm.empty[st]));
          }
          if (++st == kSt) st = 0, ph ^= 1u;
        }
        if (!ok) break;
        // the accumulator is complete once every MMA so far has retired
        if (CTAS == 1) {
          tc_commit(smem_u32(&sm.acc_full[buf]));
        } else {
          tc_commit_pair(smem_u32(&sm.acc_full[buf]));
        }
      }
    }
  } else {
    // ---- epilogue: warps 2..9; the warp's index modulo 4 selects its TMEM lane quarter, its group the column half ----
    const int quarter = warp & 3;
    const int cb = ((warp - 2) >> 2) * (BN / 2);  // first of this thread's 128 columns inside the tile
    const int row_in_tile = quarter * 32 + lane;
    const int et = tid - 64;  // 0..255
    int local = 0;
    for (int t = tile0; t < n_tiles; t += tile_step, local++) {
      const int buf = local & 1;
      int mt, nt;
      tile_coords(t, tiles_m, tiles_n, a.group_m, mt, nt);
      const int m0 = mt * BM * CTAS + int(rank) * BM, n0 = nt * TN;
      // stage this tile's bias and act(gate) slices; the barrier (id 1, the epilogue warps) also
      // separates them from the previous tile's readers
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      for (int c = et; c < BN; c += kEpiThreads) {
        // accumulator column c -> projection column: EPI_SWIGLU keeps the up half N columns further along
        const int64_t col = EPI == EPI_SWIGLU ? n0 + (c & (TN - 1)) + (c >= TN ? a.N : 0) : n0 + c;
        const bool in = EPI == EPI_SWIGLU ? n0 + (c & (TN - 1)) < a.N : col < a.N;
        sm.bias[c] = (a.bias && in) ? a.bias[col] : 0.f;
        if (EPI == EPI_RESIDUAL) {
          float gp = 1.f, gt = 1.f;
          if (a.gate.target && in) {
            gt = a.gate.target[col];
            gp = a.gate.prefix ? a.gate.prefix[col] : gt;
            if (a.gate_tanh) gt = tanhf(gt), gp = tanhf(gp);
          }
          sm.gate[0][c] = gp, sm.gate[1][c] = gt;
        }
        if (EPI == EPI_QKV && c < kHeadDim) {
          const float* nw = a.norm_w[n0 / (a.H * kHeadDim)];
          sm.gate[0][c] = nw ? nw[c] : 1.f;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      if (EPI == EPI_RESIDUAL) {
        // While the tile's main loop is still running: pull this thread's part of its row of x (512 bytes) towards L2,
        // so that the epilogue's loads, four dependent round trips per tile otherwise, find it there.
        const int64_t prow = int64_t(m0) + row_in_tile;
        if (prow < a.M) {
          const char* xr = reinterpret_cast<const char*>(a.x + prow * a.N + n0 + cb);
          for (int j = 0; j < BN / 2 * 4 / 128; j++)
            if (n0 + cb + 32 * j < a.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(xr + 128 * j));
        }
      }
      // the warps agree on the outcome of the wait, so that none is left alone at the next named barrier
      const bool landed = mbar_wait(smem_u32(&sm.acc_full[buf]), unsigned((local >> 1) & 1));
      if (!epilogue_all(landed)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int64_t row = int64_t(m0) + row_in_tile;
      const bool row_on = row < a.M;
      const unsigned taddr = tmem_base + (unsigned(quarter * 32) << 16) + unsigned(buf * kAccCols);
      // this warp is done reading the accumulator (the pair's `acc_empty` is the first CTA's)
      auto release = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CTAS == 1) mbar_arrive_local(smem_u32(&sm.acc_empty[buf]));
          else mbar_arrive_cluster(map_to_cta(smem_u32(&sm.acc_empty[buf]), 0));
        }
      };
      if constexpr (EPI == EPI_QKV) {
        // The tile's 256 columns are two heads of one tensor; this thread holds one token's row of one of them.
        // One pass over the accumulator takes each value the way the separate calls would have read it from memory -
        // bf16(acc), then bf16(. + bias) - keeps it as packed bf16 pairs (64 registers) and sums the squares.  The
        // accumulator is handed back right after that pass; normalising, rotating and storing run from registers
        // while the tensor cores fill it again.
        const int inner = a.H * kHeadDim;
        const int ti = n0 / inner, h = (n0 - ti * inner + cb) / kHeadDim;
        const bool has_norm = a.norm_w[ti] != nullptr;
        const int mode = a.mode[ti], rot = mode == MXK_ROPE_NONE ? 0 : a.rot[ti];
        unsigned P[kHeadDim / 2];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < kHeadDim; c += 16) {
          float acc[16];
          tc_ld16(taddr + unsigned(cb + c), acc);
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            float v0 = __bfloat162float(__float2bfloat16(acc[i])), v1 = __bfloat162float(__float2bfloat16(acc[i + 1]));
            if (a.bias) {
              v0 = __bfloat162float(__float2bfloat16(v0 + sm.bias[cb + c + i]));
              v1 = __bfloat162float(__float2bfloat16(v1 + sm.bias[cb + c + i + 1]));
            }
            ss = fmaf(v0, v0, ss);
            ss = fmaf(v1, v1, ss);
            P[(c + i) >> 1] = (__float_as_uint(v0) >> 16) | (__float_as_uint(v1) & 0xffff0000u);  // both are bf16 values
          }
        }
        release();
        if (row_on) {
          const float rstd = has_norm ? rsqrtf(ss * (1.f / kHeadDim) + a.eps) : 1.f;
          bf16* orow = a.out[ti] + (row * a.H + h) * kHeadDim;
          const int half = rot >> 1;
          const float* cr = a.cos + row * half;
          const float* sr = a.sin + row * half;
          if (mode == MXK_ROPE_HALF && rot > 0) {
            switch (rot >> 5) {  // rot is a multiple of 32 in this mode
              case 1: qkv_head_store<1>(P, has_norm, rstd, sm.gate[0], cr, sr, rot, orow); break;
              case 2: qkv_head_store<2>(P, has_norm, rstd, sm.gate[0], cr, sr, rot, orow); break;
              case 3: qkv_head_store<3>(P, has_norm, rstd, sm.gate[0], cr, sr, rot, orow); break;
              default: qkv_head_store<4>(P, has_norm, rstd, sm.gate[0], cr, sr, rot, orow); break;
            }
          } else {
            qkv_head_store<0>(P, has_norm, rstd, sm.gate[0], cr, sr, rot, orow);
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // This thread's 64 output columns: gate from accumulator columns [oc, oc + 64), up from [128 + oc, ...); each
        // value as silu_mul would have read it from memory (bf16(acc), then bf16(. + bias)), then the stand-alone
        // kernel's own arithmetic and rounding (act_math.cuh).
        const int oc = cb / 2;
#pragma unroll 1
        for (int c = oc; c < oc + TN / 2; c += 16) {
          float g[16], u[16];
          tc_ld16(taddr + unsigned(c), g);  // warp-wide: every lane takes part whether or not its row exists
          tc_ld16(taddr + unsigned(TN + c), u);
          if (!row_on || n0 + c >= a.N) continue;
          uint4* orow = reinterpret_cast<uint4*>(a.y + row * a.N + n0 + c);
#pragma unroll
          for (int h8 = 0; h8 < 2; h8++) {
            float gv[8], uv[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
              gv[i] = __bfloat162float(__float2bfloat16(g[8 * h8 + i]));
              uv[i] = __bfloat162float(__float2bfloat16(u[8 * h8 + i]));
              if (a.bias) gv[i] += sm.bias[c + 8 * h8 + i], uv[i] += sm.bias[TN + c + 8 * h8 + i];  // rounded by pack8
            }
            orow[h8] = act8<ACT_SILU_MUL>(pack8(gv), pack8(uv));
          }
        }
        release();
      } else {
#pragma unroll 1
        for (int c0 = cb; c0 < cb + BN / 2; c0 += 32) {
          float acc[32];
          tc_ld32(taddr + unsigned(c0), acc);  // warp-wide: every lane takes part whether or not its row exists
          if (n0 + c0 >= a.N) continue;  // the same for the whole warp (N is a multiple of 32)
          if (EPI == EPI_RESIDUAL) {
            // A thread holds 32 columns of ONE row; updating x from there would touch 32 different 128-byte lines per
            // warp instruction (measured: this epilogue then bounds the kernel, 152 us against 113 us with a bf16 store
            // on 8704 x 3072 x 3072).  So the warp turns its 32 x 32 values through shared memory: each lane writes its
            // row of y as bf16 (y IS a bf16 value: bf16(acc), then bf16(. + bias)), then the warp walks the tile four
            // rows per instruction, eight lanes on the 128 contiguous bytes of x each row has in this chunk.
            unsigned char* tile = sm.turn[warp - 2];
            uint4* mine = reinterpret_cast<uint4*>(tile + lane * kTurnRow);
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; i++) {
                float v = __bfloat162float(__float2bfloat16(acc[8 * j + i]));  // the GEMM's bf16 output
                if (a.bias) v += sm.bias[c0 + 8 * j + i];                      // add_bias_bf16: rounded by pack8
                o[i] = v;
              }
              mine[j] = pack8(o);
            }
            __syncwarp();
            const int sub = lane >> 3, c4 = (lane & 7) * 4;
            const int64_t first = int64_t(m0) + quarter * 32 + sub;
            float4 xv[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const int64_t r = first + 4 * j;
              if (r < a.M) xv[j] = *reinterpret_cast<const float4*>(a.x + r * a.N + n0 + c0 + c4);
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const int64_t r = first + 4 * j;
              if (r < a.M) {
                const uint2 yv = *reinterpret_cast<const uint2*>(tile + (sub + 4 * j) * kTurnRow + c4 * 2);
                const float* gg = sm.gate[r < a.gate.prefix_len ? 0 : 1] + c0 + c4;
                float4 o = xv[j];
                o.x = fmaf(bf16_lo(yv.x), gg[0], o.x);  // gated_residual
                o.y = fmaf(bf16_hi(yv.x), gg[1], o.y);
                o.z = fmaf(bf16_lo(yv.y), gg[2], o.z);
                o.w = fmaf(bf16_hi(yv.y), gg[3], o.w);
                *reinterpret_cast<float4*>(a.x + r * a.N + n0 + c0 + c4) = o;
              }
            }
            __syncwarp();  // the tile is rewritten by the next chunk
          } else if (row_on) {
            uint4* yr = reinterpret_cast<uint4*>(a.y + row * a.N + n0 + c0);
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; i++) {
                float v = __bfloat162float(__float2bfloat16(acc[8 * j + i]));
                if (a.bias) v += sm.bias[c0 + 8 * j + i];
                o[i] = v;
              }
              uint4 packed = pack8(o);
              if (a.act == 1) packed = act8<ACT_GELU_TANH>(packed, packed);
              else if (a.act == 2) packed = act8<ACT_GELU_ERF>(packed, packed);
              yr[j] = packed;
            }
          }
        }
        release();
      }
    }
  }

  if (!ok && a.err) atomicExch(a.err, kErrBulkTimeout);
  tc_fence_before();
  // Every role's waits are bounded, so all threads arrive here.  After a failure the producer gives the
  // copies of its last kStages fills a bounded chance to land before the CTA (and its shared memory) goes.
  const bool any_failed = __syncthreads_or(!ok) != 0;
  if (any_failed && tid == 0 && (CTAS == 1 || rank == 0)) {
    for (long it = issued > kSt ? issued - kSt : 0; it < issued; it++)
      mbar_wait(smem_u32(&sm.full[it % kSt]), unsigned((it / kSt) & 1));
  }
  if (any_failed) __syncthreads();
  if (CTAS == 2) {
    // Hand-shake of the pair: each CTA tells the other that it will signal into it no more (its epilogue and its
    // copies are done) and waits, bounded, for the same word from the other before it frees and leaves.
    if (tid == 0) {
      mbar_arrive_cluster(map_to_cta(smem_u32(&sm.done), rank ^ 1u));
      if (!mbar_wait(smem_u32(&sm.done), 0) && a.err) atomicExch(a.err, kErrBulkTimeout);
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    if (CTAS == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static std::atomic<EncodeFn> cached{nullptr};
  EncodeFn f = cached.load(std::memory_order_acquire);
  if (f) return f;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return nullptr;
  }
  f = reinterpret_cast<EncodeFn>(p);
  cached.store(f, std::memory_order_release);
  return f;
}

// bf16 [rows, K] row-major, boxes of box_rows x 64 elements, 128-byte swizzle; out-of-range parts of a box read as 0.
int make_map(const char* name, CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(MXK_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available from this driver", name);
  const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(K) * 2};
  const cuuint32_t box[2] = {cuuint32_t(BK), cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MXK_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with code %d", name, int(r));
  return MXK_OK;
}

template <int EPI, int CTAS>
int launch_linear(const char* name, const mxk_bf16* A, const mxk_bf16* W, const LinearArgs& a, cudaStream_t s);

template <int EPI>
int run_linear(const char* name, const mxk_bf16* A, const mxk_bf16* W, LinearArgs a, cudaStream_t s) {
  if (a.M <= 0) return MXK_OK;
  if (!A || !W) return fail(MXK_ERR_INVALID_ARG, "%s: null A or W", name);
  if (a.N <= 0 || a.K <= 0 || a.N % 32 != 0 || a.K % 8 != 0 || a.M >= (int64_t(1) << 31) || a.N >= (int64_t(1) << 31) ||
      a.K >= (int64_t(1) << 31))
    return fail(MXK_ERR_INVALID_ARG, "%s: need N %% 32 == 0 and K %% 8 == 0 (N=%lld K=%lld)", name, (long long)a.N, (long long)a.K);
  if (!aligned(A, 16) || !aligned(W, 16) || !aligned(a.bias, 16) || !aligned(a.x, 16) || !aligned(a.y, 16) ||
      !aligned(a.gate.target, 16) || !aligned(a.gate.prefix, 16))
    return fail(MXK_ERR_INVALID_ARG, "%s: every pointer must be 16-byte aligned", name);
  if (a.gate.target && !a.gate.prefix && a.gate.prefix_len > 0)
    return fail(MXK_ERR_INVALID_ARG, "%s: prefix_len > 0 with a null prefix vector", name);
  a.err = device_error_word();
  // Two CTAs per tile (a cluster of two, half of the W tile each) or one.  A pair tile of 256 x 256 takes about 0.9 of
  // the time of the two 128 x 256 tiles it replaces (less operand traffic), but pairs quantise the work more coarsely:
  // the form that needs fewer (weighted) waves over the SMs runs.  `linear_ctas` = 1 / 2 forces a form.
  const int want = tune(TUNE_LINEAR_CTAS, 0);
  const int64_t col_tiles = ceil_div(a.N, kTileCols<EPI>);
  const int64_t waves1 = ceil_div(ceil_div(a.M, BM) * col_tiles, int64_t(sm_count()));
  const int64_t waves2 = ceil_div(ceil_div(a.M, 2 * BM) * col_tiles, int64_t(sm_count() / 2));
  const bool pair = a.M > BM && want != 1 && (want == 2 || 9 * waves2 <= 10 * waves1);
  // band height of the tile order: a wave of 74 pairs as 8 x 9 tiles of 256 x 256, of 148 CTAs as 16 x 9 tiles of 128 x 256
  a.group_m = tune(TUNE_LINEAR_GROUP_M, pair ? 8 : 16);
  if (a.group_m < 1) a.group_m = 1;
  return pair ? launch_linear<EPI, 2>(name, A, W, a, s) : launch_linear<EPI, 1>(name, A, W, a, s);
}

template <int EPI, int CTAS>
int launch_linear(const char* name, const mxk_bf16* A, const mxk_bf16* W, const LinearArgs& a, cudaStream_t s) {
  CUtensorMap map_a, map_w;
  if (int rc = make_map(name, &map_a, A, a.M, a.K, BM)) return rc;
  // EPI_SWIGLU: W has 2 N rows (gate rows, then up rows) and is always fetched in boxes of 128 rows
  if (int rc = make_map(name, &map_w, W, EPI == EPI_SWIGLU ? 2 * a.N : a.N, a.K, EPI == EPI_SWIGLU ? BN / 2 : BN / CTAS)) return rc;
  auto k = linear_epilogue_kernel<EPI, CTAS>;
  const size_t smem = sizeof(LinearSmem<CTAS>) + 1024;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "%s: cudaFuncSetAttribute: %s", name, cudaGetErrorString(e));
  const int64_t tiles = ceil_div(a.M, BM * CTAS) * ceil_div(a.N, kTileCols<EPI>);
  int64_t units = sm_count() / CTAS;  // CTAs, or pairs of CTAs
  if (units > tiles) units = tiles;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(units * CTAS)), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute at[2];
  int n_at = 0;
  if (pdl_enabled()) {
    at[n_at].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n_at].val.programmaticStreamSerializationAllowed = 1;
    n_at++;
  }
  if (CTAS == 2) {
    at[n_at].id = cudaLaunchAttributeClusterDimension;
    at[n_at].val.clusterDim.x = 2, at[n_at].val.clusterDim.y = 1, at[n_at].val.clusterDim.z = 1;
    n_at++;
  }
  cfg.attrs = at, cfg.numAttrs = unsigned(n_at);
  cudaLaunchKernelEx(&cfg, k, map_a, map_w, a);  // errors surface through cudaGetLastError() in after_launch()
  return after_launch(name);
}

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int mxk_linear_bf16(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t N, int64_t K, mxk_bf16* y,
                    mxk_stream_t stream) {
  if (M > 0 && !y) return fail(MXK_ERR_INVALID_ARG, "linear_bf16: null y");
  LinearArgs a{};
  a.M = M, a.N = N, a.K = K, a.bias = bias, a.y = reinterpret_cast<bf16*>(y);
  return run_linear<EPI_STORE>("linear_bf16", A, W, a, as_stream(stream));
}

int mxk_linear_act(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t N, int64_t K, int act_mode,
                   mxk_bf16* y, mxk_stream_t stream) {
  if (act_mode != 0 && act_mode != 2)
    return fail(MXK_ERR_INVALID_ARG, "linear_act: act_mode %d (0 gelu tanh, 2 gelu erf; silu_mul has mxk_linear_silu_mul)", act_mode);
  if (M > 0 && !y) return fail(MXK_ERR_INVALID_ARG, "linear_act: null y");
  LinearArgs a{};
  a.M = M, a.N = N, a.K = K, a.bias = bias, a.y = reinterpret_cast<bf16*>(y), a.act = act_mode == 0 ? 1 : 2;
  return run_linear<EPI_STORE>("linear_act", A, W, a, as_stream(stream));
}

int mxk_linear_silu_mul(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t F, int64_t K, mxk_bf16* out,
                        mxk_stream_t stream) {
  if (M > 0 && !out) return fail(MXK_ERR_INVALID_ARG, "linear_silu_mul: null out");
  if (F >= (int64_t(1) << 30)) return fail(MXK_ERR_TOO_LARGE, "linear_silu_mul: F=%lld", (long long)F);
  LinearArgs a{};
  a.M = M, a.N = F, a.K = K, a.bias = bias, a.y = reinterpret_cast<bf16*>(out);
  return run_linear<EPI_SWIGLU>("linear_silu_mul", A, W, a, as_stream(stream));
}

int mxk_linear_qkv_norm_rope(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t K, int H, int D,
                             const MxkHeadTensor* tensors_host, int n_tensors, float eps, const float* cos, const float* sin,
                             mxk_stream_t stream) {
  const char* name = "linear_qkv_norm_rope";
  if (M <= 0 || n_tensors == 0) return MXK_OK;
  if (!tensors_host || n_tensors < 0 || n_tensors > 3) return fail(MXK_ERR_INVALID_ARG, "%s: n_tensors=%d (1..3)", name, n_tensors);
  if (D != kHeadDim || H <= 0 || (int64_t(H) * D) % BN != 0)
    return fail(MXK_ERR_INVALID_ARG, "%s: needs D = 128 and an even head count (H=%d D=%d); otherwise call mxk_linear_bf16 and "
                "mxk_qkv_norm_rope", name, H, D);
  LinearArgs a{};
  a.M = M, a.N = int64_t(n_tensors) * H * D, a.K = K, a.bias = bias, a.H = H, a.eps = eps, a.cos = cos, a.sin = sin;
  for (int i = 0; i < n_tensors; i++) {
    const MxkHeadTensor& t = tensors_host[i];
    if (!t.out || !aligned(t.out, 16) || !aligned(t.norm_w, 16)) return fail(MXK_ERR_INVALID_ARG, "%s: tensor %d: null or unaligned out / norm_w", name, i);
    if (t.mode != MXK_ROPE_NONE && t.mode != MXK_ROPE_INTERLEAVED && t.mode != MXK_ROPE_HALF)
      return fail(MXK_ERR_INVALID_ARG, "%s: unknown rope mode %d", name, t.mode);
    const bool rope = t.mode != MXK_ROPE_NONE && t.rot > 0;
    if (rope && (t.rot > D || t.rot % (t.mode == MXK_ROPE_HALF ? 32 : 16) != 0))
      return fail(MXK_ERR_INVALID_ARG, "%s: rot=%d must be a multiple of %d and <= D", name, t.rot, t.mode == MXK_ROPE_HALF ? 32 : 16);
    if (rope && (!cos || !sin || !aligned(cos, 16) || !aligned(sin, 16)))
      return fail(MXK_ERR_INVALID_ARG, "%s: rotary mode needs 16-byte aligned cos and sin tables", name);
    a.norm_w[i] = t.norm_w, a.out[i] = reinterpret_cast<bf16*>(t.out), a.rot[i] = rope ? t.rot : 0, a.mode[i] = rope ? t.mode : MXK_ROPE_NONE;
    // one table serves every rotating tensor of the call: they must agree on its row length
    for (int j = 0; j < i; j++)
      if (a.rot[j] && a.rot[i] && a.rot[j] != a.rot[i]) return fail(MXK_ERR_INVALID_ARG, "%s: tensors rotate %d and %d channels", name, a.rot[j], a.rot[i]);
  }
  return run_linear<EPI_QKV>(name, A, W, a, as_stream(stream));
}

int mxk_linear_gated_residual(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t N, int64_t K, float* x,
                              MxkRowMod gate, int gate_tanh, mxk_stream_t stream) {
  if (M > 0 && !x) return fail(MXK_ERR_INVALID_ARG, "linear_gated_residual: null x");
  LinearArgs a{};
  a.M = M, a.N = N, a.K = K, a.bias = bias, a.x = x, a.gate = gate, a.gate_tanh = gate_tanh;
  return run_linear<EPI_RESIDUAL>("linear_gated_residual", A, W, a, as_stream(stream));
}

}  // extern "C"
