// silu_mul, gelu_tanh_inplace, gelu_erf_inplace, silu_inplace_f32
// (reference: src/kernels/ops.cu:121-128, 212-233, 244-246).
#include "act_math.cuh"
#include "blockscale_math.cuh"
#include "flat_map.cuh"
#include "stream_pipe.cuh"

namespace mxk {
namespace {

template <int KIND>  // 0 gelu tanh, 1 gelu erf
struct GeluOp {
  static constexpr int VEC = 8;
  using Frag = uint4;
  bf16* x;
  bool vector_ok() const { return aligned(x, 16); }
  __device__ static float f(float v) { return KIND == 0 ? gelu_tanh_f(v) : gelu_erf_f(v); }
  __device__ Frag load(int64_t vi) const { return ld_stream(reinterpret_cast<const uint4*>(x) + vi); }
  __device__ void finish(int64_t vi, const Frag& r) const {
    float v[8];
    unpack8(r, v);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = f(v[i]);
    st_stream(reinterpret_cast<uint4*>(x) + vi, pack8(v));
  }
  __device__ void scalar(int64_t i) const { x[i] = __float2bfloat16(f(bf16_to_f(x[i]))); }
};

struct SiluF32Op {
  static constexpr int VEC = 4;
  using Frag = float4;
  float* x;
  bool vector_ok() const { return aligned(x, 16); }
  __device__ static float f(float v) { return v / (1.f + __expf(-v)); }
  __device__ Frag load(int64_t vi) const { return reinterpret_cast<const float4*>(x)[vi]; }
  __device__ void finish(int64_t vi, const Frag& r) const {
    reinterpret_cast<float4*>(x)[vi] = make_float4(f(r.x), f(r.y), f(r.z), f(r.w));
  }
  __device__ void scalar(int64_t i) const { x[i] = f(x[i]); }
};

// GELU in place over a flat array, for the streaming pipeline: chunk i is bytes [i*chunk, ...).
template <int KIND>
struct GeluPipeOp {
  static constexpr int NSRC = 1;
  unsigned char* x;
  int64_t nbytes;
  int chunk_bytes;
  __device__ void locate(int64_t chunk, Chunk& c) const {
    const int64_t off = chunk * chunk_bytes;
    c.src0 = x + off, c.src1 = nullptr, c.dst = x + off;
    c.bytes = unsigned(nbytes - off < chunk_bytes ? nbytes - off : chunk_bytes);
  }
  __device__ uint4 apply(const uint4& a, const uint4&) const { return act8<KIND>(a, a); }
};

// silu(gate) * up for the streaming pipeline: a row of gu is cut into chunks_per_row column chunks.
struct SiluPipeOp {
  static constexpr int NSRC = 2;
  const unsigned char* gu;
  unsigned char* out;
  int64_t F;
  int chunks_per_row, chunk_elems;
  __device__ void locate(int64_t chunk, Chunk& c) const {
    const int64_t row = chunk / chunks_per_row;
    const int64_t col = (chunk - row * chunks_per_row) * chunk_elems;
    const int64_t n = F - col < chunk_elems ? F - col : chunk_elems;
    c.src0 = gu + (row * 2 * F + col) * 2;
    c.src1 = c.src0 + F * 2;
    c.dst = out + (row * F + col) * 2;
    c.bytes = unsigned(n * 2);
  }
  __device__ uint4 apply(const uint4& g, const uint4& u) const { return act8<ACT_SILU_MUL>(g, u); }
};

// Bias add and activation in one pass: out[r, c] = act(bf16(in[r, c] + bias[c])) (GELU, in place), or
// silu(bf16(gu[r, c] + bias[c])) * bf16(gu[r, F + c] + bias[F + c]).  Chunk = a piece of one row, so
// the column of every vector is known; the bias vector is read through L1/L2.
template <int ACT>
struct BiasActPipeOp : RowPieces {
  static constexpr int NSRC = ACT == ACT_SILU_MUL ? 2 : 1;
  const float* bias;  // may be null: the plain activation
  unsigned char* out;
  float* amax;        // may be null; else max |out| is folded into it (cleared by the launcher)
  struct State {
    uint32_t m;  // two running bf16 maxima
  };
  __device__ State init() const { return State{0u}; }
  __device__ void consume(State& st, int64_t chunk, const unsigned char* stage, int tid, int n_cons) const {
    unsigned row;
    int k0, n;
    where(chunk, row, k0, n);
    const uint4* s0 = reinterpret_cast<const uint4*>(stage);
    const uint4* s1 = reinterpret_cast<const uint4*>(stage + stage_off);
    uint4* dst = reinterpret_cast<uint4*>(out + (int64_t(row) * K + k0) * 2);
    const int nvec = n >> 3;
    uint32_t m = st.m;
    for (int i = tid; i < nvec; i += n_cons) {
      uint4 g = s0[i], u = NSRC == 2 ? s1[i] : g;
      if (bias) {
        g = add_bias8(g, bias + k0 + 8 * i);
        u = NSRC == 2 ? add_bias8(u, bias + K + k0 + 8 * i) : g;
      }
      const uint4 r = act8<ACT>(g, u);
      st_stream(dst + i, r);
      if (amax) m = absmax_bf16x2(m, absmax_bf16x2(r));
    }
    st.m = m;
  }
  __device__ void finish(State& st, int) const {
    if (amax) amax_commit(bf16x2_max_to_float(st.m), amax);
  }
};

// bias (optional) + activation with ONE tile per CTA and as many CTAs as that takes: CTA (r, t) owns U x blockDim
// vectors of row r; in [rows, F] (or [rows, 2F] for silu_mul: gate then up), out [rows, F] (may be `in` for the GELUs).
template <int ACT, int U>
__global__ void __launch_bounds__(256)
    bias_act_tile_kernel(const bf16* in, const float* __restrict__ bias, int64_t F, int nvec, bf16* out) {
  constexpr bool TWO = ACT == ACT_SILU_MUL;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t r = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(in + r * F * (TWO ? 2 : 1));
  const uint4* up = g + nvec;
  uint4* o = reinterpret_cast<uint4*>(out + r * F);
  const int T = blockDim.x, base = int(blockIdx.y) * T * U + threadIdx.x;
  uint4 a[U], b[U];
#pragma unroll
  for (int k = 0; k < U; k++) {
    const int v = base + k * T;
    if (v < nvec) {
      a[k] = ld_stream(g + v);
      b[k] = TWO ? ld_stream(up + v) : a[k];
    }
  }
#pragma unroll
  for (int k = 0; k < U; k++) {
    const int v = base + k * T;
    if (v < nvec) {
      if (bias) {
        a[k] = add_bias8(a[k], bias + 8 * v);
        if (TWO) b[k] = add_bias8(b[k], bias + F + 8 * v);
      }
      st_stream(o + v, act8<ACT>(a[k], TWO ? b[k] : a[k]));
    }
  }
}

template <int ACT>
int run_bias_act(const char* name, const mxk_bf16* in, const float* bias, int64_t rows, int64_t F, mxk_bf16* out,
                 cudaStream_t s, float* amax = nullptr) {
  const bool two = ACT == ACT_SILU_MUL;
  if (F <= 0 || F % 8 != 0 || F > (int64_t(1) << 24) || !aligned(in, 16) || !aligned(out, 16) || !aligned(bias, 16))
    return fail(MXK_ERR_INVALID_ARG, "%s: needs F %% 8 == 0, F <= 2^24 and 16-byte aligned buffers; otherwise call "
                "the separate ops", name);
  if (!amax && tune(TUNE_ACT_PATH, 3) != 1 && rows < (int64_t(1) << 31)) {
    // default when no tensor maximum is asked for: one tile per CTA (as silu_mul_tile_kernel); act_path = 1 keeps the
    // pipeline below, which the maximum-producing form always takes (its running maximum lives in the consumer warps)
    const int nvec = int(F / 8);
    int threads = 256, unroll = 2, best = 1 << 30;
    for (int u = 2; u >= 1; u--)
      for (int t = 256; t >= 128; t -= 32) {
        const int tile = t * u, waste = int(ceil_div(nvec, tile)) * tile - nvec;
        if (waste < best) best = waste, threads = t, unroll = u;
      }
    const dim3 grid(unsigned(rows), unsigned(ceil_div(nvec, threads * unroll)));
    const bf16* ib = reinterpret_cast<const bf16*>(in);
    bf16* ob = reinterpret_cast<bf16*>(out);
    if (unroll == 2) launch_pdl(bias_act_tile_kernel<ACT, 2>, grid, dim3(threads), 0, s, ib, bias, F, nvec, ob);
    else launch_pdl(bias_act_tile_kernel<ACT, 1>, grid, dim3(threads), 0, s, ib, bias, F, nvec, ob);
    return after_launch(name);
  }
  int chunk_bytes = tune(TUNE_STREAM_CHUNK_KB, 8) * 1024 / (two ? 2 : 1);
  if (chunk_bytes > 32 * 1024) chunk_bytes = 32 * 1024;
  const int pieces = int(ceil_div(F * 2, chunk_bytes));
  const int piece_elems = int(ceil_div(ceil_div(F, pieces), 128) * 128);
  if (piece_elems * 2 > chunk_bytes || rows * pieces >= (int64_t(1) << 31))
    return fail(MXK_ERR_TOO_LARGE, "%s: %lld rows of %lld do not fit the pipeline's chunking", name, (long long)rows, (long long)F);
  BiasActPipeOp<ACT> op;
  op.x = reinterpret_cast<const unsigned char*>(in), op.ldx_bytes = F * (two ? 4 : 2), op.K = int(F);
  op.set_pieces(int(ceil_div(F, piece_elems)), piece_elems);
  op.src1_off = two ? F * 2 : 0, op.stage_off = (piece_elems * 2 + 127) & ~127;
  op.bias = bias, op.out = reinterpret_cast<unsigned char*>(out), op.amax = amax;
  return run_stream_pipe(name, op, rows * op.pieces_per_row, piece_elems * 2, s, two ? 4 : 8, two ? 2 : 3);
}

template <int KIND>
int run_gelu(const char* name, mxk_bf16* x, int64_t n, cudaStream_t s) {
  bf16* xb = reinterpret_cast<bf16*>(x);
  const int64_t body = n / 8 * 8;
  // Default: the flat kernel, two vectors per thread, ONE tile per CTA and as many CTAs as that takes.  On B200 that
  // beats both persistent forms - a resident wave of the same kernel walking the array grid-stride, and the bulk-copy
  // pipeline below (8 consumer warps, 3 stages of 8 KB): 63.3 us against 79.5 and 74.5 us on 107 M elements in
  // place.  The hardware scheduler hands out tiles as SMs free up, so there is no ramp and no tail, and 2048
  // threads per SM with two loads each keep more bytes in flight than the pipeline's stages.  act_path = 1 keeps
  // the pipeline selectable.
  if (tune(TUNE_ACT_PATH, 2) == 1 && aligned(x, 16) && body >= (int64_t(1) << 16)) {
    const int chunk_bytes = tune(TUNE_STREAM_CHUNK_KB, 8) * 1024;
    GeluPipeOp<KIND> op{reinterpret_cast<unsigned char*>(x), body * 2, chunk_bytes};
    if (int rc = run_stream_pipe(name, op, ceil_div(body * 2, chunk_bytes), chunk_bytes, s, 8, 3)) return rc;
    if (n > body) {  // fewer than 8 ragged elements at the end
      flat_scalar_kernel<GeluOp<KIND>><<<1, 32, 0, s>>>(n - body, GeluOp<KIND>{xb + body});
      return after_launch(name);
    }
    return MXK_OK;
  }
  return run_flat(name, n, GeluOp<KIND>{xb}, s, 2, true);
}

constexpr int kActRowsInFlight = 4;

// out[r, c] = silu(gu[r, c]) * gu[r, F + c]; each thread owns 8 columns and walks a strip of rows.
__global__ void __launch_bounds__(256)
    silu_mul_kernel(const bf16* __restrict__ gu, int64_t rows, int F, bf16* __restrict__ out,
                    int rows_per_chunk) {
  constexpr int U = kActRowsInFlight;
  pdl_launch_dependents();
  pdl_wait();
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (col >= F) return;
  const int64_t nchunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
  for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const int64_t r0 = c * rows_per_chunk;
    const int64_t r1 = r0 + rows_per_chunk < rows ? r0 + rows_per_chunk : rows;
    for (int64_t r = r0; r < r1; r += U) {
      uint4 g[U], u[U];
#pragma unroll
      for (int k = 0; k < U; k++) {
        if (r + k < r1) {
          const bf16* p = gu + (r + k) * 2 * F + col;
          g[k] = ld_stream(reinterpret_cast<const uint4*>(p));
          u[k] = ld_stream(reinterpret_cast<const uint4*>(p + F));
        }
      }
#pragma unroll
      for (int k = 0; k < U; k++) {
        if (r + k < r1) {
          float a[8], b[8];
          unpack8(g[k], a);
          unpack8(u[k], b);
#pragma unroll
          for (int i = 0; i < 8; i++) a[i] = silu_f(a[i]) * b[i];
          st_stream(reinterpret_cast<uint4*>(out + (r + k) * F + col), pack8(a));
        }
      }
    }
  }
}

// The same op with ONE tile per CTA and as many CTAs as that takes: CTA (r, t) owns U x blockDim vectors of row r;
// every thread has 2 U independent loads in flight and there is no loop.
template <int U>
__global__ void __launch_bounds__(256)
    silu_mul_tile_kernel(const bf16* __restrict__ gu, int64_t F, int nvec, bf16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t r = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(gu + r * 2 * F);
  const uint4* up = g + nvec;
  uint4* o = reinterpret_cast<uint4*>(out + r * F);
  const int T = blockDim.x, base = int(blockIdx.y) * T * U + threadIdx.x;
  uint4 a[U], b[U];
#pragma unroll
  for (int k = 0; k < U; k++) {
    const int v = base + k * T;
    if (v < nvec) a[k] = ld_stream(g + v), b[k] = ld_stream(up + v);
  }
#pragma unroll
  for (int k = 0; k < U; k++) {
    const int v = base + k * T;
    if (v < nvec) st_stream(o + v, act8<ACT_SILU_MUL>(a[k], b[k]));
  }
}

__global__ void __launch_bounds__(256)
    silu_mul_scalar_kernel(const bf16* __restrict__ gu, int64_t rows, int F, bf16* __restrict__ out) {
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= F) return;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float g = bf16_to_f(gu[row * 2 * F + i]);
    const float u = bf16_to_f(gu[row * 2 * F + F + i]);
    out[row * F + i] = __float2bfloat16(silu_f(g) * u);
  }
}

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int mxk_bias_gelu_tanh_inplace(mxk_bf16* x, const float* bias, int64_t rows, int64_t F, mxk_stream_t stream) {
  if (rows <= 0 || F <= 0) return MXK_OK;
  if (!x) return fail(MXK_ERR_INVALID_ARG, "bias_gelu_tanh_inplace: null x");
  if (!bias) return mxk_gelu_tanh_inplace(x, rows * F, stream);
  return run_bias_act<ACT_GELU_TANH>("bias_gelu_tanh_inplace", x, bias, rows, F, x, as_stream(stream));
}

int mxk_bias_silu_mul(const mxk_bf16* gu, const float* bias, int64_t rows, int64_t F, mxk_bf16* out, mxk_stream_t stream) {
  if (rows <= 0 || F <= 0) return MXK_OK;
  if (!gu || !out) return fail(MXK_ERR_INVALID_ARG, "bias_silu_mul: null gu or out");
  if (!bias) return mxk_silu_mul(gu, rows, F, out, stream);
  return run_bias_act<ACT_SILU_MUL>("bias_silu_mul", gu, bias, rows, F, out, as_stream(stream));
}

int mxk_act_amax(int act_mode, const mxk_bf16* in, const float* bias, int64_t rows, int64_t F, mxk_bf16* out, float* amax_out,
                 mxk_stream_t stream) {
  if (!amax_out) return fail(MXK_ERR_INVALID_ARG, "act_amax: null amax_out");
  if (act_mode < 0 || act_mode > 2) return fail(MXK_ERR_INVALID_ARG, "act_amax: act_mode %d (0 gelu tanh, 1 silu_mul, 2 gelu erf)", act_mode);
  cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), as_stream(stream));
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "act_amax: cudaMemsetAsync: %s", cudaGetErrorString(e));
  if (rows <= 0 || F <= 0) return MXK_OK;
  if (!in || !out) return fail(MXK_ERR_INVALID_ARG, "act_amax: null in or out");
  cudaStream_t s = as_stream(stream);
  if (act_mode == 1) return run_bias_act<ACT_SILU_MUL>("act_amax", in, bias, rows, F, out, s, amax_out);
  if (act_mode == 0) return run_bias_act<ACT_GELU_TANH>("act_amax", in, bias, rows, F, out, s, amax_out);
  return run_bias_act<ACT_GELU_ERF>("act_amax", in, bias, rows, F, out, s, amax_out);
}

int mxk_silu_mul(const mxk_bf16* gu, int64_t rows, int64_t F, mxk_bf16* out, mxk_stream_t stream) {
  if (rows <= 0 || F <= 0) return MXK_OK;
  if (!gu || !out) return fail(MXK_ERR_INVALID_ARG, "silu_mul: null gu or out");
  if (F > (int64_t(1) << 29)) return fail(MXK_ERR_INVALID_ARG, "silu_mul: F=%lld out of range", (long long)F);
  cudaStream_t s = as_stream(stream);
  const bf16* in = reinterpret_cast<const bf16*>(gu);
  bf16* o = reinterpret_cast<bf16*>(out);
  if (tune(TUNE_ACT_PATH, 3) == 3 && F % 8 == 0 && aligned(gu, 16) && aligned(out, 16) && rows < (int64_t(1) << 31) &&
      F / 8 <= 65535 * 128) {  // grid.y holds the tiles of a row
    // Default: one tile per CTA, as many CTAs as that takes (33272 x 13824: 413 us against 426 us for the bulk-copy
    // pipeline below and 523 us for the register kernel on one resident wave; 33272 x 14336: 428 / 465 us).
    // tile = threads x U vectors, chosen so that the row is a whole number of tiles if one of the shapes allows it
    const int nvec = int(F / 8);
    int threads = 256, unroll = 2, best = 1 << 30;
    for (int u = 2; u >= 1; u--)
      for (int t = 256; t >= 128; t -= 32) {
        const int tile = t * u, waste = int(ceil_div(nvec, tile)) * tile - nvec;
        if (waste < best) best = waste, threads = t, unroll = u;
      }
    const dim3 grid(unsigned(rows), unsigned(ceil_div(nvec, threads * unroll)));
    if (unroll == 2) launch_pdl(silu_mul_tile_kernel<2>, grid, dim3(threads), 0, s, in, F, nvec, o);
    else launch_pdl(silu_mul_tile_kernel<1>, grid, dim3(threads), 0, s, in, F, nvec, o);
    return after_launch("silu_mul");
  }
  if (tune(TUNE_ACT_PATH, 3) == 1 && F % 8 == 0 && aligned(gu, 16) && aligned(out, 16) && rows * F >= (int64_t(1) << 16)) {
    const int chunk_bytes = tune(TUNE_STREAM_CHUNK_KB, 4) * 1024;  // 4 warps, 2 stages of 2 x 4 KB measured best
    int cpr = int(ceil_div(F * 2, chunk_bytes));
    int chunk_elems = int(ceil_div(ceil_div(F, cpr), 8) * 8);
    int warps = 4;
    // The pipeline's loop-free path needs chunks of exactly two vectors per consumer thread (64 vectors per warp).  A row
    // that is not a whole number of 4 KB chunks (13824 columns = 6.75 of them) is cut into equal chunks that are, on as
    // many warps as that takes: 13824 columns = 3 chunks of 9 KB on nine warps, 424.6 us against 434.1 us on 33272 rows.
    const int64_t row_vecs = F / 8;
    if (row_vecs % 256 != 0 && tune(TUNE_STREAM_CHUNK_KB, 0) == 0 && tune(TUNE_STREAM_WARPS, 0) == 0) {
      for (int wv = 12; wv >= 5; wv--)
        if (row_vecs % (64 * wv) == 0) {
          warps = wv, chunk_elems = 64 * wv * 8, cpr = int(F / chunk_elems);
          break;
        }
    }
    SiluPipeOp op{reinterpret_cast<const unsigned char*>(gu), reinterpret_cast<unsigned char*>(out), F, cpr, chunk_elems};
    return run_stream_pipe("silu_mul", op, rows * cpr, chunk_elems * 2, s, warps, 2);
  }
  if (F % 8 == 0 && aligned(gu, 16) && aligned(out, 16)) {
    const int threads = 256;
    const int rpc = tune(TUNE_ACT_ROWS_PER_CTA, 4);
    const unsigned gy = unsigned(ceil_div(F / 8, threads));
    const int64_t nchunks = ceil_div(rows, rpc);
    int64_t gx = ceil_div(int64_t(sm_count()) * resident_ctas(silu_mul_kernel, threads), gy);
    if (gx > nchunks) gx = nchunks;
    if (gx < 1) gx = 1;
    launch_pdl(silu_mul_kernel, dim3(unsigned(gx), gy), dim3(threads), 0, s, in, rows, int(F), o, rpc);
  } else {
    const unsigned gy = unsigned(ceil_div(F, 256));
    int64_t gx = rows < int64_t(sm_count()) * 16 ? rows : int64_t(sm_count()) * 16;
    silu_mul_scalar_kernel<<<dim3(unsigned(gx), gy), 256, 0, s>>>(in, rows, int(F), o);
  }
  return after_launch("silu_mul");
}

int mxk_gelu_tanh_inplace(mxk_bf16* x, int64_t n, mxk_stream_t stream) {
  if (n <= 0) return MXK_OK;
  if (!x) return fail(MXK_ERR_INVALID_ARG, "gelu_tanh_inplace: null x");
  return run_gelu<0>("gelu_tanh_inplace", x, n, as_stream(stream));
}

int mxk_gelu_erf_inplace(mxk_bf16* x, int64_t n, mxk_stream_t stream) {
  if (n <= 0) return MXK_OK;
  if (!x) return fail(MXK_ERR_INVALID_ARG, "gelu_erf_inplace: null x");
  return run_gelu<1>("gelu_erf_inplace", x, n, as_stream(stream));
}

int mxk_silu_inplace_f32(float* x, int64_t n, mxk_stream_t stream) {
  if (n <= 0) return MXK_OK;
  if (!x) return fail(MXK_ERR_INVALID_ARG, "silu_inplace_f32: null x");
  return run_flat("silu_inplace_f32", n, SiluF32Op{x}, as_stream(stream));
}

}  // extern "C"
