/*
 * mxk.h - C ABI of libmxk, the sm_100a implementation of Miroxen's fused DiT layer ops.
 *
 * Every entry point below replaces one launcher of the reference's src/kernels/ops.h (the
 * citation beside each declaration is the reference declaration it stands in for) or one of the
 * host-side table builders in its model graphs.  The conventions are the reference's own:
 *
 *  - all data pointers are caller-owned DEVICE memory on the CURRENT device, unless the
 *    parameter name ends in _host;
 *  - the call is asynchronous on `stream`; nothing here synchronises, allocates, frees or
 *    changes the current device;
 *  - rows <= 0 / S <= 0 / n <= 0 is a silent no-op that returns MXK_OK (src/kernels/ops.cu:155,
 *    179, 200, 139);
 *  - bf16 tensors are passed as uint16_t* holding the raw bfloat16 bit patterns;
 *  - the residual stream is fp32, GEMM/attention operands are bf16, modulation vectors, norm
 *    weights and cos/sin tables are fp32, arithmetic is fp32 (src/kernels/ops.h:2).
 *
 * Return value: MXK_OK (0) or a negative MXK_ERR_* code; mxk_last_error() then returns a
 * thread-local, human-readable message.  The C++ shim in mx_ops.h turns a non-zero status into
 * std::runtime_error, which is what the reference's MX_CHECK / MX_KCHECK macros throw
 * (src/core/common.h:34-48).
 */
#ifndef MXK_H_
#define MXK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXK_OK 0
#define MXK_ERR_INVALID_ARG (-1) /* a shape, pointer or mode the op cannot accept */
#define MXK_ERR_CUDA (-2)        /* the CUDA runtime reported an error at launch */
#define MXK_ERR_TOO_LARGE (-3)   /* a size beyond a documented fixed limit */

typedef uint16_t mxk_bf16;  /* raw bfloat16 bits */
typedef void* mxk_stream_t; /* a cudaStream_t */

/* Per-row choice between two modulation vectors: rows with index < prefix_len use `prefix`,
 * the others `target`; target == NULL means "this modulation is absent".  Same layout as the
 * reference's RowMod (src/kernels/ops.h:11-15). */
typedef struct MxkRowMod {
  const float* target;
  const float* prefix;
  int64_t prefix_len;
} MxkRowMod;

/* src/kernels/ops.h:39 enum RopeMode */
#define MXK_ROPE_NONE 0
#define MXK_ROPE_INTERLEAVED 1 /* channel pairs (2i, 2i+1) */
#define MXK_ROPE_HALF 2        /* channel pairs (i, i + rot/2) */

const char* mxk_last_error(void);
/* ABI version of the library (major * 100 + minor). */
int mxk_version(void);
/* Number of kernel launches this thread has issued through the library since the last call of
 * mxk_reset_launch_count(); used by the benchmark to state its own launch count. */
int64_t mxk_launch_count(void);
void mxk_reset_launch_count(void);

/* ---- normalisation + modulation + cast -------------------------------------------------- */

/* src/kernels/ops.h:18 layernorm_mod: out = bf16(LayerNorm(x) * (1 + scale) + shift), no affine,
 * two-pass variance, rstd = rsqrt(var + eps). x fp32 [rows, dim], out bf16 [rows, dim]. */
int mxk_layernorm_mod(const float* x, int64_t rows, int64_t dim, float eps, MxkRowMod scale,
                      MxkRowMod shift, mxk_bf16* out, mxk_stream_t stream);
/* src/kernels/ops.h:21 rmsnorm_mod: out = bf16(x * rsqrt(mean(x^2) + eps) * w * (1 + scale) + shift);
 * w, scale and shift may each be absent. */
int mxk_rmsnorm_mod(const float* x, int64_t rows, int64_t dim, float eps, const float* w,
                    MxkRowMod scale, MxkRowMod shift, mxk_bf16* out, mxk_stream_t stream);
/* src/kernels/ops.h:24 rmsnorm_bf16: rmsnorm_mod with a bf16 input and no modulation. */
int mxk_rmsnorm_bf16(const mxk_bf16* x, int64_t rows, int64_t dim, float eps, const float* w,
                     mxk_bf16* out, mxk_stream_t stream);

/* No counterpart in the reference (its launchers have one kernel per op).  Reports which kernel
 * family a norm call with these pointer values and sizes would take: 0 = one CTA per row (any
 * size / alignment), 1 = register row kernel (8/16-byte vector accesses), 2 = bulk-copy row kernel
 * (rows copied to shared memory with cp.async.bulk, which needs every row of x, and of y in the
 * fused forms, to start on a 16-byte boundary).  op: 0 layernorm_mod, 1 rmsnorm_mod,
 * 2 rmsnorm_bf16, 3 / 4 gated_residual_norm with LayerNorm / RMSNorm, 5 / 6 the same two with
 * MXFP8 output (`out` stands for q; these return 2 or MXK_ERR_INVALID_ARG, as the entry point
 * would).  Pure host arithmetic: nothing is dereferenced and no CUDA call is made, so it works
 * without a GPU. */
int mxk_norm_path_probe(int op, const void* x, const void* y, const void* out, const float* w, MxkRowMod scale,
                        MxkRowMod shift, MxkRowMod gate, int64_t rows, int64_t dim);

/* ---- residual --------------------------------------------------------------------------- */

/* src/kernels/ops.h:27 gated_residual: x += act(gate) * y with act = tanh when gate_tanh != 0,
 * identity otherwise; gate.target == NULL gives x += y. x fp32 [rows, dim], y bf16 [rows, dim]. */
int mxk_gated_residual(float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate,
                       int gate_tanh, mxk_stream_t stream);
/* src/kernels/ops.h:30 add_inplace_bf16: x(bf16) = bf16(x + y). */
int mxk_add_inplace_bf16(mxk_bf16* x, const mxk_bf16* y, int64_t n, mxk_stream_t stream);

/* ---- per-head RMSNorm + rotary ---------------------------------------------------------- */

/* src/kernels/ops.h:35 head_norm_rope: head h of token s is in[s*in_stride + col0 + h*D .. +D);
 * optional per-head RMSNorm (norm_w fp32 [D], NULL skips it) then rotary on the first `rot`
 * channels with cos/sin fp32 [S, rot/2]; writes out bf16 [S, H, D].  D even and <= 256, rot even
 * and <= D (src/kernels/ops.cu:201).  mode MXK_ROPE_NONE with norm_w == NULL is a strided copy. */
int mxk_head_norm_rope(const mxk_bf16* in, int64_t S, int64_t in_stride, int64_t col0, int H,
                       int D, const float* norm_w, float eps, const float* cos, const float* sin,
                       int rot, int mode, mxk_bf16* out, mxk_stream_t stream);

/* ---- activations ------------------------------------------------------------------------ */

/* src/kernels/ops.h:44 silu_mul: gu bf16 [rows, 2F] (gate | up) -> out bf16 [rows, F] = silu(gate) * up. */
int mxk_silu_mul(const mxk_bf16* gu, int64_t rows, int64_t F, mxk_bf16* out, mxk_stream_t stream);
/* src/kernels/ops.h:46 gelu_tanh_inplace: x = bf16(0.5 v (1 + tanh(0.7978845608 (v + 0.044715 v^3)))). */
int mxk_gelu_tanh_inplace(mxk_bf16* x, int64_t n, mxk_stream_t stream);
/* src/kernels/ops.h:48 gelu_erf_inplace: x = bf16(0.5 v (1 + erf(v / sqrt 2))). */
int mxk_gelu_erf_inplace(mxk_bf16* x, int64_t n, mxk_stream_t stream);
/* src/kernels/ops.h:51 silu_inplace_f32: x = x / (1 + exp(-x)) on fp32. */
int mxk_silu_inplace_f32(float* x, int64_t n, mxk_stream_t stream);

/* ---- helpers around the GEMMs ----------------------------------------------------------- */

/* src/kernels/ops.h:50 scatter_rows: x[rows[i], :] = src[i, :] (+= when add != 0); rows int32 [n]
 * on the device, x fp32 [*, dim], src bf16 [n, dim]. */
int mxk_scatter_rows(float* x, int64_t dim, const int32_t* rows, const mxk_bf16* src, int64_t n,
                     int add, mxk_stream_t stream);
/* src/kernels/ops.h:53 add_bias_bf16: y[r, :] = bf16(y[r, :] + bias). */
int mxk_add_bias_bf16(mxk_bf16* y, const float* bias, int64_t rows, int64_t dim, mxk_stream_t stream);
/* src/kernels/ops.h:54 add_bias_f32 */
int mxk_add_bias_f32(float* y, const float* bias, int64_t rows, int64_t dim, mxk_stream_t stream);
/* src/kernels/ops.h:56 f32_to_bf16 */
int mxk_f32_to_bf16(const float* x, mxk_bf16* y, int64_t n, mxk_stream_t stream);
/* src/kernels/ops.h:57 bf16_to_f32 */
int mxk_bf16_to_f32(const mxk_bf16* x, float* y, int64_t n, mxk_stream_t stream);
/* src/kernels/ops.h:59 axpy_f32: x += a * y */
int mxk_axpy_f32(float* x, const float* y, float a, int64_t n, mxk_stream_t stream);
/* src/kernels/ops.h:61 axpby_f32: x = a * x + b * y */
int mxk_axpby_f32(float* x, const float* y, float a, float b, int64_t n, mxk_stream_t stream);

/* ---- fused extensions (no single counterpart in ops.h; each equals the two or three
 *      reference calls named, issued back to back on the same rows) ------------------------ */

/* gated_residual (src/kernels/ops.h:27) followed by layernorm_mod / rmsnorm_mod
 * (src/kernels/ops.h:18,21) on the same rows, as src/models/qwen_image/dit.cpp:305-307 and
 * src/models/minimax_h3/dit.cpp:238-239 call them: x is read once, updated in place and
 * normalised from registers.  norm_mode 0 = LayerNorm, 1 = RMSNorm. */
int mxk_gated_residual_norm(float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate,
                            int gate_tanh, int norm_mode, float eps, const float* w,
                            MxkRowMod scale, MxkRowMod shift, mxk_bf16* out, mxk_stream_t stream);

/* One tensor of a multi-tensor head_norm_rope launch. */
typedef struct MxkHeadTensor {
  const mxk_bf16* in; /* [S, in_stride] */
  int64_t in_stride;
  int64_t col0;
  const float* norm_w; /* fp32 [D] or NULL */
  mxk_bf16* out;       /* [S, H, D] */
  int rot;             /* 0 with mode NONE = copy */
  int mode;
} MxkHeadTensor;
/* Up to three head_norm_rope calls (q, k and the v copy of src/models/minimax_h3/dit.cpp:210-213;
 * q and k of src/models/qwen_image/dit.cpp:270-272) that share S, H, D, eps and the cos/sin table,
 * in one launch: the token's cos/sin row is fetched once for all of them. */
int mxk_qkv_norm_rope(const MxkHeadTensor* tensors_host, int n_tensors, int64_t S, int H, int D,
                      float eps, const float* cos, const float* sin, mxk_stream_t stream);

/* ---- head exchange for sequence parallelism --------------------------------------------- */
/* The reference's 2-card path (src/models/minimax_h3/dit_sp.cpp:83-112) shards token rows for the
 * linear layers and attention heads for attention: after the QKV projection each card runs
 * head_norm_rope once per card on that card's head range into a send buffer and copies it over
 * (cudaMemcpyPeerAsync), so that every card ends with [S, H/2 * D] = all rows, its own heads.  Here
 * that is one launch for any G <= MXK_MAX_HEAD_GROUPS: the q / k / v heads of this rank's `S` rows
 * are normalised and rotated exactly as mxk_qkv_norm_rope does and head h of tensor i is stored
 * straight into outs_host[i * groups + h / (H / groups)], a bf16 [*, H / groups, D] array, at row
 * dst_row0 + s.  A destination may be a peer GPU's buffer (mxk_peer_buffer_open): the stores then
 * cross NVLink and no send buffer or copy exists.  Stores are plain per-lane 128-bit stores; the
 * kernel waits on nobody.  The caller orders the consumers of the destinations after every rank's
 * launch (an event per peer as in dit_sp.cpp:111,116, or a barrier).  tensors[i].out is ignored.
 * H must be a multiple of groups; D one of 32, 64, 128, 256; inputs 16-byte aligned. */
#define MXK_MAX_HEAD_GROUPS 8
int mxk_qkv_norm_rope_scatter(const MxkHeadTensor* tensors_host, int n_tensors, int64_t S, int H, int D, float eps,
                              const float* cos, const float* sin, int groups, mxk_bf16* const* outs_host,
                              int64_t dst_row0, mxk_stream_t stream);
/* The way back (src/models/minimax_h3/dit_sp.cpp:137-149): rows [src_row0, src_row0 + rows) of the
 * attention output are gathered from the `groups` head-sharded arrays srcs_host[g] (bf16
 * [*, heads_per_group, D], this GPU's or a peer's: plain 128-bit loads) into out bf16
 * [rows, groups * heads_per_group * D], the input layout of the out-projection. */
int mxk_gather_head_groups(const mxk_bf16* const* srcs_host, int groups, int64_t src_row0, int64_t rows,
                           int heads_per_group, int D, mxk_bf16* out, mxk_stream_t stream);
/* Set-up helpers for the peer buffers (they allocate; never on the hot path).  alloc: cudaMalloc on
 * the current device + an opaque 64-byte handle another process of the same box passes to open,
 * which maps the buffer into its address space and enables peer access (CUDA IPC).  close undoes
 * open; free releases an allocation of alloc. */
int mxk_peer_buffer_alloc(int64_t bytes, void** ptr, unsigned char* handle64);
int mxk_peer_buffer_open(const unsigned char* handle64, void** ptr);
int mxk_peer_buffer_close(void* ptr);
int mxk_peer_buffer_free(void* ptr);


/* ---- linear layers with the following op in the GEMM epilogue ------------------------------- */
/* The reference's linear() is a library GEMM that stores a bf16 matrix, followed by add_bias_bf16 as a
 * read-modify-write of it (src/core/weights.cpp:159-177); the attention out-projection and the second
 * MLP projection are then consumed by gated_residual (src/models/qwen_image/dit.cpp:304-305,313-314;
 * src/models/minimax_h3/dit.cpp:238,245).  These entry points run the GEMM on the tensor cores
 * (tcgen05.mma, accumulator in tensor memory, operands by TMA) and apply those ops in the epilogue with
 * the reference's roundings, y = bf16(acc), y = bf16(y + bias), so the results are what the separate
 * calls give up to the accumulation order of the GEMM.
 *   A bf16 [M, K] row-major, W bf16 [N, K] row-major (the [out, in] weight layout), bias fp32 [N] or
 *   NULL.  N % 32 == 0, K % 8 == 0, every pointer 16-byte aligned.
 * mxk_linear_bf16:            y bf16 [M, N] = A W^T (+ bias)              = linear()
 * mxk_linear_gated_residual:  x fp32 [M, N] += act(gate) * (A W^T (+ bias)) = linear() + gated_residual()
 * mxk_linear_qkv_norm_rope:   the QKV projection with head_norm_rope in its epilogue: W bf16
 *   [n_tensors * H * 128, K] (the q | k | v rows of the packed projection, src/models/minimax_h3/dit.cpp:207-213;
 *   three separate projections can be passed as one concatenated weight), bias fp32 [n_tensors * H * 128] or
 *   NULL; tensors_host[i] gives tensor i's norm_w (NULL: none), rot, mode and out (bf16 [M, H, 128]); its in,
 *   in_stride and col0 are ignored.  = linear() + head_norm_rope() per tensor, the [M, 3 H D] projection
 *   output never written.  D must be 128 and H even; rot a multiple of 16 (interleaved) or 32 (half).
 * mxk_linear_act:             y bf16 [M, N] = act(A W^T (+ bias)), act_mode 0 GELU (tanh form) / 2 GELU (erf form)
 *   = linear() + gelu_tanh_inplace() (src/models/qwen_image/dit.cpp:192-193), one write instead of a write and
 *   a read-modify-write.
 * mxk_linear_silu_mul:        out bf16 [M, F] = silu(g) * u with [g | u] = A W^T (+ bias), W bf16 [2 F, K] (gate rows,
 *   then up rows: the reference's concatenated gate_up weight), bias fp32 [2 F] or NULL.  = linear(gate_up) +
 *   silu_mul() (src/models/qwen_image/dit.cpp:309-312, src/models/minimax_h3/dit.cpp:241-242); the [M, 2 F]
 *   projection is never written.  F % 32 == 0.
 * No counterpart as single calls in the reference (each replaces two or three of its calls). */
int mxk_linear_qkv_norm_rope(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t K, int H, int D,
                             const MxkHeadTensor* tensors_host, int n_tensors, float eps, const float* cos, const float* sin,
                             mxk_stream_t stream);
int mxk_linear_act(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t N, int64_t K, int act_mode,
                   mxk_bf16* y, mxk_stream_t stream);
int mxk_linear_silu_mul(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t F, int64_t K, mxk_bf16* out,
                        mxk_stream_t stream);
int mxk_linear_bf16(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t N, int64_t K, mxk_bf16* y,
                    mxk_stream_t stream);
int mxk_linear_gated_residual(const mxk_bf16* A, const mxk_bf16* W, const float* bias, int64_t M, int64_t N, int64_t K, float* x,
                              MxkRowMod gate, int gate_tanh, mxk_stream_t stream);

/* ---- RoPE tables and timestep embeddings ------------------------------------------------
 * The reference builds these on the host with libm and uploads them once per generation
 * (src/models/qwen_image/dit.cpp:151-185, src/models/minimax_h3/dit.cpp:254-262).  libm's
 * cosf/sinf are not reproducible by a different algorithm, so bit-exact tables need libm.  The
 * split used here: the host evaluates libm only on the DISTINCT (position, frequency) pairs of
 * each axis (a few thousand values), and a kernel expands those per-axis look-up tables into
 * the [S, rot/2] table by each row's position index. */

/* Describes a run of consecutive rows whose per-axis look-up indices follow a grid:
 * row r = row0 + (i0 * n1 + i1) * n2 + i2 with i0 < n0, i1 < n1, i2 < n2 has, on axis a,
 * the look-up index base[a] + i0*step0[a] + i1*step1[a] + i2*step2[a]. */
typedef struct MxkRopeRun {
  int64_t row0;
  int32_t n0, n1, n2;
  int32_t base[3];
  int32_t step0[3];
  int32_t step1[3];
  int32_t step2[3];
} MxkRopeRun;

/* Expand per-axis look-up tables into cos/sin fp32 [S, half].  lut_cos/lut_sin: device fp32,
 * axis a occupies rows [lut_row0[a], ...) of width pairs[a] starting at element lut_off[a];
 * output pair columns of axis a are [col0[a], col0[a] + pairs[a]).  runs_host: n_runs
 * descriptors (<= 64) covering [0, S). */
int mxk_rope_table_expand(const float* lut_cos, const float* lut_sin, const int64_t* lut_off_host,
                          const int32_t* pairs_host, const int32_t* col0_host, int n_axes,
                          const MxkRopeRun* runs_host, int n_runs, int64_t S, int half, float* cos,
                          float* sin, mxk_stream_t stream);

/* Host builders (pure host code, libm; they touch no GPU).  Each returns MXK_OK or an error. */

/* MSRoPE inverse frequencies of src/models/qwen_image/dit.cpp:153-157:
 * invf = 1.0f / powf(theta, float(2j) / float(axis)) for each axis in turn; out_host has
 * sum(axes[a] / 2) entries. */
int mxk_msrope_inv_freq_host(const int32_t* axes_host, int n_axes, float theta, float* out_host);
/* Look-up table of one axis: lut[(p - pos_min) * pairs + j] = cosf/sinf(float(p) * invf[j]) for
 * p in [pos_min, pos_max] (src/models/qwen_image/dit.cpp:160-166). */
int mxk_rope_lut_int_host(int64_t pos_min, int64_t pos_max, const float* invf_host, int pairs,
                          float* lut_cos_host, float* lut_sin_host);
/* Same for explicit fp32 positions (src/models/minimax_h3/dit.cpp:258-262):
 * lut[i * pairs + j] = cosf/sinf(pos[i] * invf[j]). */
int mxk_rope_lut_f32_host(const float* pos_host, int64_t n, const float* invf_host, int pairs,
                          float* lut_cos_host, float* lut_sin_host);
/* Spatial rotary coordinates of one latent axis (src/models/minimax_h3/layout.cpp:15-21):
 * g[k] = float(((1 - r)/2 + r*k/n) * 32) with r = dim / sqrt(H*W), n = dim/2, in double. */
int mxk_h3_spatial_grid_host(int64_t dim, int64_t H, int64_t W, float* out_host);
/* Time coordinate of each latent frame (src/models/minimax_h3/layout.cpp:90-97):
 * ft[f] = T + sum_{g<f} (5/3) * {1,4,4,4,4}[g % 5], in double, returned as fp32. */
int mxk_h3_frame_times_host(int64_t T, int64_t F_lat, float* out_host);
/* Qwen-Image timestep embedding (src/models/qwen_image/dit.cpp:220-230): two rows (t and 0) of
 * 256 values, cos half first, t and every value rounded through bf16. out_host fp32 [2, 256]. */
int mxk_qwen_timestep_embedding_host(float t, float* out_host);
/* The same embedding evaluated on the device: frequencies come from libm on the host, the
 * angle is the same fp32 product, cos/sin are evaluated in fp64 and rounded to fp32 then bf16.
 * out fp32 [2, 256] on the device. */
int mxk_qwen_timestep_embedding(float t, float* out, mxk_stream_t stream);
/* MiniMax-H3 time basis (src/models/minimax_h3/dit.cpp:166-179): linear interpolation in
 * table fp32 [grid, basis] at pos = clamp(t, 0, 1) * (grid - 1); ts fp32 [nt] and table on the
 * device, out fp32 [nt, basis].  Uses unfused multiply and add so the result is bit-identical
 * to the host formula. */
int mxk_h3_time_basis(const float* ts, int64_t nt, const float* table, int64_t grid, int64_t basis,
                      float* out, mxk_stream_t stream);

/* ---- call-pattern drivers ---------------------------------------------------------------
 * The op sequence the reference's model graphs issue around each GEMM / attention call, with
 * the GEMM and attention outputs supplied by the caller as ready-made device buffers. */

typedef struct MxkBlockArgs {
  /* Shapes: rows tokens; residual width dim; attention width inner = H * D; MLP width F. */
  int64_t rows, dim, F;
  int H, D;
  int norm_mode; /* 0 LayerNorm (no affine), 1 RMSNorm */
  float eps;
  int act_mode;  /* 0: gelu_tanh_inplace on act [rows, F]; 1: silu_mul of act2 [rows, 2F] into act */
  int fused;     /* 0: one launch per reference call; 1: the fused extensions where calls are adjacent */
  int64_t chunk_rows; /* > 0: issue the sequence per chunk of this many rows (src/models/minimax_h3/dit.cpp:199) */
  /* Modulation (each may have target == NULL) and RMSNorm weights (NULL = none). */
  const float* norm1_w;
  const float* norm2_w;
  MxkRowMod shift1, scale1, gate1, shift2, scale2, gate2;
  int gate_tanh;
  /* q / k / v projections: head h of row s is X_in[s * qkv_stride + X_col0 + h * D ...]. v_in NULL = no v. */
  const mxk_bf16* q_in;
  const mxk_bf16* k_in;
  const mxk_bf16* v_in;
  int64_t qkv_stride, q_col0, k_col0, v_col0;
  const float* norm_q; /* fp32 [D] */
  const float* norm_k;
  const float* cos; /* fp32 [rows, rot/2] */
  const float* sin;
  int rot, rope_mode;
  mxk_bf16* q_out; /* bf16 [rows, H, D] */
  mxk_bf16* k_out;
  mxk_bf16* v_out;
  /* Residual stream and the GEMM-side buffers. */
  float* x;               /* fp32 [rows, dim], updated in place */
  mxk_bf16* h1;           /* bf16 [rows, dim], first norm output (input of the QKV GEMM) */
  mxk_bf16* h2;           /* bf16 [rows, dim], second norm output (input of the MLP GEMM); may equal h1 */
  const mxk_bf16* attn_o; /* bf16 [rows, dim], stand-in for the attention out-projection */
  mxk_bf16* act;          /* bf16 [rows, F] */
  const mxk_bf16* act2;   /* bf16 [rows, 2F] when act_mode == 1 */
  const mxk_bf16* mlp_o;  /* bf16 [rows, dim], stand-in for the MLP down-projection */
} MxkBlockArgs;
/* The fused-op sequence of one DiT block in the order of src/models/qwen_image/dit.cpp:265-314 and
 * src/models/minimax_h3/dit.cpp:199-247: norm+mod, q/k(/v) head norm + rope, gated residual,
 * norm+mod, activation, gated residual. */
int mxk_dit_block_ops(const MxkBlockArgs* a, mxk_stream_t stream);

/* Measurement aid: only the first n_ops launches of that sequence (chunk_rows must be 0).  Timing the
 * prefixes 1, 2, ... of a block and taking differences gives each op's cost inside the chain with the
 * launches still overlapping as they do in mxk_dit_block_ops (events between the launches would
 * serialise them). */
int mxk_dit_block_ops_prefix(const MxkBlockArgs* a, int n_ops, mxk_stream_t stream);

/* Per-op device timing of one mxk_dit_block_ops pass: a CUDA event is recorded on the stream before
 * the first op and after every op.  The handle owns 16 events (created here, not on the hot path). */
typedef struct MxkOpTimes MxkOpTimes;
int mxk_op_times_create(MxkOpTimes** out);
void mxk_op_times_destroy(MxkOpTimes* t);
/* Same launches as mxk_dit_block_ops (chunk_rows must be 0) with the events in between. */
int mxk_dit_block_ops_timed(const MxkBlockArgs* a, mxk_stream_t stream, MxkOpTimes* t);
/* Waits for the last event of the most recent timed pass and writes the milliseconds of each op, in
 * launch order, to ms_host; returns the number of ops (>= 0) or a negative status. */
int mxk_op_times_read(MxkOpTimes* t, float* ms_host, int cap);

/* The same sequence with HOST buffers: rows are streamed through the GPU in chunks, the copies
 * of one chunk overlapping the kernels of another on three internal streams owned by the handle.
 * Host buffers should be pinned for the copies to overlap. */
typedef struct MxkHostPipeline MxkHostPipeline;
/* Allocates MXK_HOST_PIPELINE_SLOTS (three) sets of device staging buffers for chunks of chunk_rows
 * rows, three streams and nine events (this is the one place the library allocates device memory; the
 * handle owns it).  Device bytes per set: chunk_rows x (4 dim + 4 x 2 dim + (4, or 6 with_v) x 2 H D +
 * 2 F (+ 4 F when act_mode == 1) + 2 x 4 max(rot / 2, 1)), each array rounded up to 256 bytes; a caller that
 * sizes an arena budgets three times that.  with_v / act_mode mirror the args. */
#define MXK_HOST_PIPELINE_SLOTS 3
int mxk_host_pipeline_create(int64_t chunk_rows, int64_t dim, int64_t F, int H, int D, int rot,
                             int with_v, int act_mode, MxkHostPipeline** out);
void mxk_host_pipeline_destroy(MxkHostPipeline* p);
/* `a` holds HOST pointers for x, h1, h2, q/k/v_in, q/k/v_out, attn_o, act, act2, mlp_o, cos, sin
 * and DEVICE pointers for the modulation vectors and norm weights; q/k/v_in are read as separate
 * [rows, H*D] arrays (qkv_stride and col0 as given apply to the host arrays).  Blocks until the
 * results are back in host memory.  h2d_bytes / d2h_bytes (may be NULL) receive the bytes copied.
 * Before returning it reads the device error word (see mxk_device_error): if a kernel's bounded wait
 * ran out during the call the status is MXK_ERR_CUDA and the host results are incomplete.  Callers of
 * the device-buffer entry points, which never synchronise, poll mxk_device_error themselves. */
int mxk_dit_block_ops_host(MxkHostPipeline* p, const MxkBlockArgs* a, int64_t* h2d_bytes,
                           int64_t* d2h_bytes);

/* No counterpart in the reference.  mxk_dit_block_ops_host for callers that must not allocate
 * device memory: code that runs after start-up inside a fixed memory budget (an engine that sized its
 * arena once and may never grow it, a plugin loaded into a host process that forbids cudaMalloc on its
 * threads) or at a point where an allocation would synchronise the whole device.  It runs the same op
 * sequence on HOST buffers, one chunk of rows at a time, on the caller's stream and without overlap
 * between copies and kernels; its device staging is a fixed array of MXK_STATIC_STAGE_MIB MiB inside
 * the library's device image (mxk_static_stage_bytes() returns the size; every GPU that loads the
 * library holds it until the process exits).  It calls no cudaMalloc / cudaFree and creates no streams
 * or events.
 *  - Limit: 64 rows of staging must fit the array (for a 3072-wide block one row stages about 85 KB);
 *    wider blocks return MXK_ERR_TOO_LARGE.  The number of rows is not limited.
 *  - The first call on each device looks the array's address up (cudaGetSymbolAddress, with that
 *    device current) and keeps it for the life of the process; make that first call before any
 *    stream capture begins.  The kept address does not survive a cudaDeviceReset of that device:
 *    after a reset the library must be reloaded before this entry point is used again.
 *  - The stream must belong to the current device (the array that is used is the current device's);
 *    a stream of another device is refused with MXK_ERR_INVALID_ARG before any copy is issued.
 *  - Like mxk_dit_block_ops_host it reads the device error word before returning and reports a
 *    kernel's timed-out wait as MXK_ERR_CUDA.
 *  - All calls on a device share the one array.  It keeps the previous call's bytes, which is harmless:
 *    every byte a chunk's kernels read is first written by that chunk's own copies or kernels, so
 *    nothing has to start at zero.  Two calls whose work overlaps on the GPU (different streams or
 *    threads) race on the array and corrupt each other's results: serialise them.
 * `a` is laid out as for mxk_dit_block_ops_host; returns after the results are in host memory. */
#define MXK_STATIC_STAGE_MIB 32
int64_t mxk_static_stage_bytes(void);
int mxk_dit_block_ops_host_static(const MxkBlockArgs* a, mxk_stream_t stream, int64_t* h2d_bytes,
                                  int64_t* d2h_bytes);

/* Reads (and with clear != 0 resets) the current device's error word: 0, or 1 when a kernel's bounded
 * wait on a bulk copy ran out and the kernel returned early (its outputs are then incomplete).
 * Synchronises with the device. */
int mxk_device_error(int* out_host, int clear);

/* Self-test of the kernels' failure path: launches one small CTA that waits, with a budget of four
 * tries (under 100 microseconds), on a barrier that is never completed; the kernel gives up, sets the
 * device error word to 1 and returns, leaving the context usable.  mxk_device_error() then reads 1. */
int mxk_selftest_bounded_wait(mxk_stream_t stream);

/* ---- activation block-scale quantiser (the step after this library's ops on the fp8 / fp4 path) ----
 *
 * Replaces quantize_blockscaled(), qdata_bytes() and qscale_bytes() of src/kernels/blockscale.h:27-43
 * (kernels at src/kernels/blockscale.cu:47-129, launcher 147-164; called on every activation by
 * src/core/weights.cpp:189-195).  x is bf16 [rows, K] with row stride ldx (elements).
 *   MXK_Q_MXFP8: q = rows * K e4m3 bytes, sf = one ue8m0 byte per 32 elements of a row.
 *   MXK_Q_NVFP4: q = rows * K / 2 bytes (two e2m1 codes per byte, low nibble first), sf = one e4m3 byte
 *                per 16 elements, *amax (device fp32, required) receives max|x|; the tensor scale the
 *                GEMM needs is amax / 2688.
 * sf has mxk_qscale_bytes() bytes in cuBLASLt's VEC32_UE8M0 / VEC16_UE4M3 layout (rows padded to 128,
 * scale columns to 4, 128 x 4 tiles interleaved) and is cleared first, padding included.
 * Requirements as the reference's: K % 32 == 0, ldx % 8 == 0, x 16-byte aligned; q 16-byte aligned.
 * Outputs are byte-identical to the reference kernel's. */
enum { MXK_Q_MXFP8 = 1, MXK_Q_NVFP4 = 2 };
int64_t mxk_qdata_bytes(int mode, int64_t rows, int64_t K);
int64_t mxk_qscale_bytes(int mode, int64_t rows, int64_t K);
int mxk_quantize_blockscaled(int mode, const mxk_bf16* x, int64_t ldx, int64_t rows, int64_t K, void* q, uint8_t* sf,
                             float* amax, mxk_stream_t stream);

/* NVFP4 without the extra read pass.  The reference's quantiser reads an NVFP4 input twice: once for
 * the tensor maximum no block can be scaled without (amax_kernel, src/kernels/blockscale.cu:47-70),
 * once to quantise (:147-164).  The op that PRODUCES the tensor can take the maximum of its own bf16
 * output as it stores it; these variants do (packed bf16 maxima per thread, one atomicMax per warp),
 * clearing *amax_out first on the same stream:
 *   mxk_layernorm_mod_amax / mxk_rmsnorm_mod_amax / mxk_gated_residual_norm_amax: the norm entry points
 *     with one more argument;
 *   mxk_act_amax: act_mode 0 GELU-tanh (out may be in: in place), 1 silu_mul (in bf16 [rows, 2F] ->
 *     out [rows, F]), 2 GELU-erf; bias (may be NULL) is added first as in mxk_bias_gelu_tanh_inplace /
 *     mxk_bias_silu_mul.
 * mxk_quantize_nvfp4_known_amax then quantises in one pass from that device value (which it only
 * reads).  Bytes (codes, scales, maximum) equal mxk_quantize_blockscaled(MXK_Q_NVFP4) on the same
 * tensor.  No single counterpart in the reference (two adjacent calls become one and a half). */
int mxk_layernorm_mod_amax(const float* x, int64_t rows, int64_t dim, float eps, MxkRowMod scale, MxkRowMod shift,
                           mxk_bf16* out, float* amax_out, mxk_stream_t stream);
int mxk_rmsnorm_mod_amax(const float* x, int64_t rows, int64_t dim, float eps, const float* w, MxkRowMod scale,
                         MxkRowMod shift, mxk_bf16* out, float* amax_out, mxk_stream_t stream);
int mxk_gated_residual_norm_amax(float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate, int gate_tanh,
                                 int norm_mode, float eps, const float* w, MxkRowMod scale, MxkRowMod shift, mxk_bf16* out,
                                 float* amax_out, mxk_stream_t stream);
int mxk_act_amax(int act_mode, const mxk_bf16* in, const float* bias, int64_t rows, int64_t F, mxk_bf16* out, float* amax_out,
                 mxk_stream_t stream);
int mxk_quantize_nvfp4_known_amax(const mxk_bf16* x, int64_t ldx, int64_t rows, int64_t K, void* q, uint8_t* sf,
                                  const float* amax, mxk_stream_t stream);

/* Activation and MXFP8 quantisation in one pass over the data, for an activation whose only reader is the
 * next block-scaled GEMM (the MLP's hidden activation).  One call in place of two of the reference's:
 * gelu_tanh_inplace / gelu_erf_inplace / silu_mul (src/kernels/ops.h:36-41) followed by
 * quantize_blockscaled(MXFP8) (src/kernels/blockscale.h:30); the bf16 activation is never written, which
 * takes the traffic from 7 bytes per element to 3.  Results are byte-identical to mxk_gelu_tanh_inplace /
 * mxk_gelu_erf_inplace / mxk_silu_mul followed by mxk_quantize_blockscaled.
 *   act_mode 0: gelu (tanh form) of in [rows, F];  1: silu(in[:, :F]) * in[:, F:] with in [rows, 2F];
 *            2: gelu (erf form) of in [rows, F].
 * bias (nullable): fp32 [F] ([2F] for act_mode 1) that linear() would have added with add_bias_bf16 right after the
 * GEMM (src/core/weights.cpp:164-167); in + bias is rounded to bf16 first, so the bits are those of the three calls.
 * F % 32 == 0, in, bias and q 16-byte aligned.  NVFP4 has no such form: its first block cannot be scaled before
 * the maximum of the whole activation is known. */
int mxk_act_quantize_mxfp8(int act_mode, const mxk_bf16* in, const float* bias, int64_t rows, int64_t F, void* q, uint8_t* sf,
                           mxk_stream_t stream);

/* Norm, modulation and MXFP8 quantisation in one pass, for a normed activation whose only readers are
 * block-scaled GEMMs.  One call in place of layernorm_mod / rmsnorm_mod (src/kernels/ops.h:22-25) followed by
 * quantize_blockscaled(MXFP8) (src/kernels/blockscale.h:30); arguments as mxk_layernorm_mod / mxk_rmsnorm_mod
 * with (q, sf) in place of the bf16 output.  The bf16 row stays in shared memory and is never written: 5 bytes
 * per element instead of 9.  Byte-identical to the two calls of this library.  dim % 32 == 0, 16-byte aligned
 * vectors and q; a shape outside the one-pass kernel returns -1 and asks for the two calls. */
int mxk_layernorm_mod_quant_mxfp8(const float* x, int64_t rows, int64_t dim, float eps, MxkRowMod scale,
                                  MxkRowMod shift, void* q, uint8_t* sf, mxk_stream_t stream);
int mxk_rmsnorm_mod_quant_mxfp8(const float* x, int64_t rows, int64_t dim, float eps, const float* w, MxkRowMod scale,
                                MxkRowMod shift, void* q, uint8_t* sf, mxk_stream_t stream);
/* The whole adjacent sequence of a block on the fp8 path in one pass: gated_residual, then the norm, then the
 * quantisation (src/models/qwen_image/dit.cpp:305-307 followed by linear()'s quantize_blockscaled): x is updated
 * in place, (q, sf) receive the MXFP8 form of the normed row; 11 bytes per element instead of 19.  Arguments as
 * mxk_gated_residual_norm with (q, sf) in place of the bf16 output; byte-identical to mxk_gated_residual_norm
 * followed by mxk_quantize_blockscaled. */
int mxk_gated_residual_norm_quant_mxfp8(float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate, int gate_tanh,
                                        int norm_mode, float eps, const float* w, MxkRowMod scale, MxkRowMod shift, void* q,
                                        uint8_t* sf, mxk_stream_t stream);

/* ---- latent layout kernels either side of the DiT ----
 *
 * mx::qwen_latent::encode / decode (src/kernels/qwen_latent.h:7-8): encode x [64, n] -> y [n, 64] as
 * (x - mean[c]) / std[c]; decode x [n, 64] -> y [64, n] as x * std[c] + mean[c]; each step rounded on
 * its own (no fused multiply-add), bit-identical to the reference.  mean, std: 64 device floats; x and y
 * must not overlap.
 * mx::h3_latent::video / audio (src/kernels/h3_latent.h:6-7): DiT rows -> the VAE's channel-first layout,
 * values untouched.  video: rows [frames * h/2 * w/2, 96] -> z [24, frames, h, w] (a row holds 24 channels
 * x 2 x 2 pixels); audio: rows [2 * samples, 32] -> z [2, 32, samples].  h and w even.
 * Unlike the layer ops, a bad argument here is an error (-1), as in the reference. */
int mxk_qwen_latent_encode(const float* x, float* y, int64_t n, const float* mean, const float* std, mxk_stream_t stream);
int mxk_qwen_latent_decode(const float* x, float* y, int64_t n, const float* mean, const float* std, mxk_stream_t stream);
int mxk_h3_latent_video(const float* rows, float* z, int64_t frames, int64_t h, int64_t w, mxk_stream_t stream);
int mxk_h3_latent_audio(const float* rows, float* z, int64_t samples, mxk_stream_t stream);

/* ---- bias add folded into the op that follows it ----
 *
 * linear() adds a layer's bias with add_bias_bf16 right after the GEMM (src/core/weights.cpp:164-167), a
 * read-modify-write of the whole output, and one of the ops above then reads that output again.  These take
 * the bias instead (the caller skips its add_bias_bf16) and read the GEMM output once; (y + bias) is rounded
 * to bf16 first, so the bits are those of mxk_add_bias_bf16 followed by the plain op.  A null bias gives the
 * plain op.  Valid when nothing else touches the output between the bias add and the op (no LoRA branch
 * accumulating into it).
 *   mxk_bias_gelu_tanh_inplace: x[r, c] = gelu_tanh(bf16(x[r, c] + bias[c])), x bf16 [rows, F], bias fp32 [F].
 *   mxk_bias_silu_mul: out[r, c] = silu(bf16(gu[r, c] + bias[c])) * bf16(gu[r, F + c] + bias[F + c]),
 *                      gu bf16 [rows, 2F], bias fp32 [2F].
 *   mxk_gated_residual_bias: x[r, :] += act(gate) * bf16(y[r, :] + bias), arguments as mxk_gated_residual.
 * F % 8 == 0 (dim % 8 == 0, dim <= 8192) and 16-byte aligned buffers; other shapes return -1 and ask for the
 * two calls. */
int mxk_bias_gelu_tanh_inplace(mxk_bf16* x, const float* bias, int64_t rows, int64_t F, mxk_stream_t stream);
int mxk_bias_silu_mul(const mxk_bf16* gu, const float* bias, int64_t rows, int64_t F, mxk_bf16* out, mxk_stream_t stream);
int mxk_gated_residual_bias(float* x, const mxk_bf16* y, const float* bias, int64_t rows, int64_t dim, MxkRowMod gate,
                            int gate_tanh, mxk_stream_t stream);

/* Development knob: overrides a launch-shape default (see tuning.h for the names); value 0
 * restores the default.  Results do not depend on it. */
int mxk_set_tuning(const char* name, int value);

#ifdef __cplusplus
}
#endif
#endif /* MXK_H_ */
