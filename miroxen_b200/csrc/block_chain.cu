// Call-pattern drivers: the sequence of fused layer ops one DiT block issues around its GEMM and
// attention calls (reference: src/models/qwen_image/dit.cpp:245-315 run_block,
// src/models/minimax_h3/dit.cpp:183-248 attn_mlp), on device buffers and - streamed in row
// chunks over three streams - on host buffers.
#include <atomic>
#include <cstring>

#include "common.cuh"

namespace mxk {
namespace {

MxkRowMod shifted(MxkRowMod m, int64_t r0) {
  // A launch that starts at row r0 sees the prefix boundary r0 rows earlier
  // (src/kernels/ops.cu:183-184).
  m.prefix_len -= r0;
  return m;
}

int check_block(const MxkBlockArgs* a) {
  if (!a) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops: null args");
  if (a->rows < 0 || a->dim <= 0 || a->F <= 0 || a->H <= 0 || a->D <= 0)
    return fail(MXK_ERR_INVALID_ARG, "dit_block_ops: rows=%lld dim=%lld F=%lld H=%d D=%d", (long long)a->rows,
                (long long)a->dim, (long long)a->F, a->H, a->D);
  if (a->norm_mode != 0 && a->norm_mode != 1) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops: norm_mode=%d", a->norm_mode);
  if (a->act_mode != 0 && a->act_mode != 1) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops: act_mode=%d", a->act_mode);
  if (!a->x || !a->h1 || !a->h2 || !a->q_in || !a->k_in || !a->q_out || !a->k_out || !a->attn_o || !a->act || !a->mlp_o)
    return fail(MXK_ERR_INVALID_ARG, "dit_block_ops: null buffer");
  if (a->act_mode == 1 && !a->act2) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops: act_mode == 1 needs act2");
  if (a->v_in && !a->v_out) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops: v_in without v_out");
  return MXK_OK;
}

// Reads the device error word behind everything already queued on `s` and waits for it.  The host-buffer
// entry points hand results back in host memory, so a kernel that gave up on a bounded wait (and left
// part of its output unwritten) must turn into a status here: nobody else would look.  The word is left
// set; mxk_device_error() reads and clears it.
int device_error_status(const char* name, cudaStream_t s) {
  int word = 0;
  int* p = device_error_word();
  if (!p) return fail(MXK_ERR_CUDA, "%s: no error word on this device", name);
  cudaError_t e = cudaMemcpyAsync(&word, p, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "%s: reading the device error word: %s", name, cudaGetErrorString(e));
  if (word != 0)
    return fail(MXK_ERR_CUDA, "%s: a kernel's bounded wait ran out (device error word = %d); the results in host memory "
                "are incomplete", name, word);
  return MXK_OK;
}

#define MXK_TRY(expr)            \
  do {                           \
    if (int rc_ = (expr)) return rc_; \
  } while (0)

// Optional per-op timing: an event is recorded on the stream before the first op and after each op.
struct OpTimer {
  cudaEvent_t* ev = nullptr;
  int cap = 0, used = 0;
  void mark(mxk_stream_t s) {
    if (ev && used < cap) cudaEventRecord(ev[used++], as_stream(s));
  }
};

// Rows [r0, r0 + n) of the block.
int block_rows(const MxkBlockArgs& a, int64_t r0, int64_t n, mxk_stream_t s, OpTimer* tm = nullptr, int max_ops = 1 << 30) {
  OpTimer none;
  OpTimer& T = tm ? *tm : none;
  T.mark(s);
  int ops_left = max_ops;
#define MXK_OP_DONE()              \
  do {                             \
    if (--ops_left <= 0) return MXK_OK; \
  } while (0)
  if (ops_left <= 0) return MXK_OK;
  const int64_t dim = a.dim, inner = int64_t(a.H) * a.D, F = a.F, half = a.rot / 2;
  float* x = a.x + r0 * dim;
  mxk_bf16* h1 = a.h1 + r0 * dim;
  mxk_bf16* h2 = a.h2 + r0 * dim;
  const float* cs = a.cos ? a.cos + r0 * half : nullptr;
  const float* sn = a.sin ? a.sin + r0 * half : nullptr;
  const MxkRowMod sc1 = shifted(a.scale1, r0), sh1 = shifted(a.shift1, r0), g1 = shifted(a.gate1, r0);
  const MxkRowMod sc2 = shifted(a.scale2, r0), sh2 = shifted(a.shift2, r0), g2 = shifted(a.gate2, r0);

  if (a.norm_mode == 0) MXK_TRY(mxk_layernorm_mod(x, n, dim, a.eps, sc1, sh1, h1, s));
  else MXK_TRY(mxk_rmsnorm_mod(x, n, dim, a.eps, a.norm1_w, sc1, sh1, h1, s));
  T.mark(s);
  MXK_OP_DONE();

  MxkHeadTensor t[3];
  int nt = 0;
  t[nt++] = MxkHeadTensor{a.q_in + r0 * a.qkv_stride, a.qkv_stride, a.q_col0, a.norm_q, a.q_out + r0 * inner, a.rot, a.rope_mode};
  t[nt++] = MxkHeadTensor{a.k_in + r0 * a.qkv_stride, a.qkv_stride, a.k_col0, a.norm_k, a.k_out + r0 * inner, a.rot, a.rope_mode};
  if (a.v_in) t[nt++] = MxkHeadTensor{a.v_in + r0 * a.qkv_stride, a.qkv_stride, a.v_col0, nullptr, a.v_out + r0 * inner, 0, MXK_ROPE_NONE};
  if (a.fused) {
    MXK_TRY(mxk_qkv_norm_rope(t, nt, n, a.H, a.D, a.eps, cs, sn, s));
    T.mark(s);
    MXK_OP_DONE();
  } else {
    for (int i = 0; i < nt; i++) {
      MXK_TRY(mxk_head_norm_rope(t[i].in, n, t[i].in_stride, t[i].col0, a.H, a.D, t[i].norm_w, i < 2 ? a.eps : 0.f,
                                 i < 2 ? cs : nullptr, i < 2 ? sn : nullptr, t[i].rot, t[i].mode, t[i].out, s));
      T.mark(s);
      MXK_OP_DONE();
    }
  }

  if (a.fused) {
    MXK_TRY(mxk_gated_residual_norm(x, a.attn_o + r0 * dim, n, dim, g1, a.gate_tanh, a.norm_mode, a.eps, a.norm2_w, sc2,
                                    sh2, h2, s));
    T.mark(s);
    MXK_OP_DONE();
  } else {
    MXK_TRY(mxk_gated_residual(x, a.attn_o + r0 * dim, n, dim, g1, a.gate_tanh, s));
    T.mark(s);
    MXK_OP_DONE();
    if (a.norm_mode == 0) MXK_TRY(mxk_layernorm_mod(x, n, dim, a.eps, sc2, sh2, h2, s));
    else MXK_TRY(mxk_rmsnorm_mod(x, n, dim, a.eps, a.norm2_w, sc2, sh2, h2, s));
    T.mark(s);
    MXK_OP_DONE();
  }

  if (a.act_mode == 0) MXK_TRY(mxk_gelu_tanh_inplace(a.act + r0 * F, n * F, s));
  else MXK_TRY(mxk_silu_mul(a.act2 + r0 * 2 * F, n, F, a.act + r0 * F, s));
  T.mark(s);
  MXK_OP_DONE();

  MXK_TRY(mxk_gated_residual(x, a.mlp_o + r0 * dim, n, dim, g2, a.gate_tanh, s));
  T.mark(s);
#undef MXK_OP_DONE
  return MXK_OK;
}

}  // namespace
}  // namespace mxk

using namespace mxk;

struct MxkOpTimes {
  cudaEvent_t ev[16];
  int cap, used;
};

// Staging slots of the host pipeline: with three, the upload of chunk c + 2 never waits for the
// download of chunk c (it reuses the slot of chunk c - 1, whose results left one chunk time earlier).
constexpr int kHostSlots = MXK_HOST_PIPELINE_SLOTS;

struct MxkHostPipeline {
  int64_t chunk_rows, dim, F, inner, half;
  int H, D, rot, with_v, act_mode;
  int device;
  cudaStream_t h2d, comp, d2h;
  struct Slot {
    char* base;
    float* x;
    mxk_bf16 *h1, *h2, *q_in, *k_in, *v_in, *q_out, *k_out, *v_out, *attn_o, *act, *act2, *mlp_o;
    float *cos, *sin;
    cudaEvent_t h2d_done, comp_done, d2h_done;
  } slot[kHostSlots];
};

extern "C" {

int mxk_dit_block_ops(const MxkBlockArgs* a, mxk_stream_t stream) {
  if (int rc = check_block(a)) return rc;
  if (a->rows == 0) return MXK_OK;
  const int64_t chunk = a->chunk_rows > 0 ? a->chunk_rows : a->rows;
  for (int64_t r0 = 0; r0 < a->rows; r0 += chunk) {
    const int64_t n = a->rows - r0 < chunk ? a->rows - r0 : chunk;
    if (int rc = block_rows(*a, r0, n, stream)) return rc;
  }
  return MXK_OK;
}

int mxk_dit_block_ops_prefix(const MxkBlockArgs* a, int n_ops, mxk_stream_t stream) {
  if (int rc = check_block(a)) return rc;
  if (a->chunk_rows > 0 && a->chunk_rows < a->rows)
    return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_prefix: covers one chunk (chunk_rows must be 0)");
  if (a->rows == 0 || n_ops <= 0) return MXK_OK;
  return block_rows(*a, 0, a->rows, stream, nullptr, n_ops);
}

int mxk_op_times_create(MxkOpTimes** out) {
  if (!out) return fail(MXK_ERR_INVALID_ARG, "op_times_create: null out");
  MxkOpTimes* t = new MxkOpTimes();
  t->cap = 16, t->used = 0;
  for (int i = 0; i < t->cap; i++) {
    cudaError_t e = cudaEventCreate(&t->ev[i]);
    if (e != cudaSuccess) {
      for (int j = 0; j < i; j++) cudaEventDestroy(t->ev[j]);
      delete t;
      return fail(MXK_ERR_CUDA, "op_times_create: %s", cudaGetErrorString(e));
    }
  }
  *out = t;
  return MXK_OK;
}

void mxk_op_times_destroy(MxkOpTimes* t) {
  if (!t) return;
  for (int i = 0; i < t->cap; i++) cudaEventDestroy(t->ev[i]);
  delete t;
}

int mxk_dit_block_ops_timed(const MxkBlockArgs* a, mxk_stream_t stream, MxkOpTimes* t) {
  if (!t) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_timed: null timer");
  if (int rc = check_block(a)) return rc;
  if (a->chunk_rows > 0 && a->chunk_rows < a->rows)
    return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_timed: per-op timing covers one chunk (chunk_rows must be 0)");
  OpTimer tm;
  tm.ev = t->ev, tm.cap = t->cap, tm.used = 0;
  t->used = 0;
  if (a->rows == 0) return MXK_OK;
  int rc = block_rows(*a, 0, a->rows, stream, &tm);
  t->used = tm.used;
  return rc;
}

int mxk_op_times_read(MxkOpTimes* t, float* ms_host, int cap) {
  if (!t || !ms_host) return fail(MXK_ERR_INVALID_ARG, "op_times_read: null argument");
  const int n = t->used > 0 ? t->used - 1 : 0;
  if (n > cap) return fail(MXK_ERR_TOO_LARGE, "op_times_read: %d intervals, room for %d", n, cap);
  if (n > 0) {
    cudaError_t e = cudaEventSynchronize(t->ev[t->used - 1]);
    if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "op_times_read: %s", cudaGetErrorString(e));
  }
  for (int i = 0; i < n; i++) {
    cudaError_t e = cudaEventElapsedTime(&ms_host[i], t->ev[i], t->ev[i + 1]);
    if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "op_times_read: %s", cudaGetErrorString(e));
  }
  return n;
}

int mxk_host_pipeline_create(int64_t chunk_rows, int64_t dim, int64_t F, int H, int D, int rot,
                             int with_v, int act_mode, MxkHostPipeline** out) {
  if (!out) return fail(MXK_ERR_INVALID_ARG, "host_pipeline_create: null out");
  *out = nullptr;
  if (chunk_rows <= 0 || dim <= 0 || F <= 0 || H <= 0 || D <= 0 || rot < 0 || rot > D)
    return fail(MXK_ERR_INVALID_ARG, "host_pipeline_create: bad shape");
  MxkHostPipeline* p = new MxkHostPipeline();
  memset(p, 0, sizeof(*p));
  p->chunk_rows = chunk_rows, p->dim = dim, p->F = F, p->H = H, p->D = D, p->rot = rot;
  p->inner = int64_t(H) * D, p->half = rot / 2, p->with_v = with_v, p->act_mode = act_mode;
  auto bail = [&](const char* what, cudaError_t e) {
    int rc = fail(MXK_ERR_CUDA, "host_pipeline_create: %s: %s", what, cudaGetErrorString(e));
    mxk_host_pipeline_destroy(p);
    return rc;
  };
  cudaError_t e;
  if ((e = cudaGetDevice(&p->device)) != cudaSuccess) return bail("cudaGetDevice", e);
  if ((e = cudaStreamCreateWithFlags(&p->h2d, cudaStreamNonBlocking)) != cudaSuccess) return bail("stream", e);
  if ((e = cudaStreamCreateWithFlags(&p->comp, cudaStreamNonBlocking)) != cudaSuccess) return bail("stream", e);
  if ((e = cudaStreamCreateWithFlags(&p->d2h, cudaStreamNonBlocking)) != cudaSuccess) return bail("stream", e);
  auto pad = [](int64_t b) { return (b + 255) / 256 * 256; };
  const int64_t R = chunk_rows;
  const int64_t bx = pad(R * dim * 4), bh = pad(R * dim * 2), bi = pad(R * p->inner * 2), bf = pad(R * F * 2),
                bf2 = act_mode == 1 ? pad(R * 2 * F * 2) : 0, bt = pad(R * (p->half > 0 ? p->half : 1) * 4);
  const int64_t total = bx + 2 * bh /*h1 h2*/ + 2 * bh /*attn_o mlp_o*/ + (with_v ? 6 : 4) * bi + bf + bf2 + 2 * bt;
  for (int i = 0; i < kHostSlots; i++) {
    MxkHostPipeline::Slot& s = p->slot[i];
    if ((e = cudaMalloc(reinterpret_cast<void**>(&s.base), size_t(total))) != cudaSuccess) return bail("cudaMalloc", e);
    char* c = s.base;
    auto take = [&](int64_t b) { char* r = c; c += b; return r; };
    s.x = reinterpret_cast<float*>(take(bx));
    s.h1 = reinterpret_cast<mxk_bf16*>(take(bh));
    s.h2 = reinterpret_cast<mxk_bf16*>(take(bh));
    s.attn_o = reinterpret_cast<mxk_bf16*>(take(bh));
    s.mlp_o = reinterpret_cast<mxk_bf16*>(take(bh));
    s.q_in = reinterpret_cast<mxk_bf16*>(take(bi));
    s.k_in = reinterpret_cast<mxk_bf16*>(take(bi));
    s.q_out = reinterpret_cast<mxk_bf16*>(take(bi));
    s.k_out = reinterpret_cast<mxk_bf16*>(take(bi));
    if (with_v) {
      s.v_in = reinterpret_cast<mxk_bf16*>(take(bi));
      s.v_out = reinterpret_cast<mxk_bf16*>(take(bi));
    }
    s.act = reinterpret_cast<mxk_bf16*>(take(bf));
    if (act_mode == 1) s.act2 = reinterpret_cast<mxk_bf16*>(take(bf2));
    s.cos = reinterpret_cast<float*>(take(bt));
    s.sin = reinterpret_cast<float*>(take(bt));
    if ((e = cudaEventCreateWithFlags(&s.h2d_done, cudaEventDisableTiming)) != cudaSuccess) return bail("event", e);
    if ((e = cudaEventCreateWithFlags(&s.comp_done, cudaEventDisableTiming)) != cudaSuccess) return bail("event", e);
    if ((e = cudaEventCreateWithFlags(&s.d2h_done, cudaEventDisableTiming)) != cudaSuccess) return bail("event", e);
  }
  *out = p;
  return MXK_OK;
}

void mxk_host_pipeline_destroy(MxkHostPipeline* p) {
  if (!p) return;
  for (int i = 0; i < kHostSlots; i++) {
    MxkHostPipeline::Slot& s = p->slot[i];
    if (s.base) cudaFree(s.base);
    if (s.h2d_done) cudaEventDestroy(s.h2d_done);
    if (s.comp_done) cudaEventDestroy(s.comp_done);
    if (s.d2h_done) cudaEventDestroy(s.d2h_done);
  }
  if (p->h2d) cudaStreamDestroy(p->h2d);
  if (p->comp) cudaStreamDestroy(p->comp);
  if (p->d2h) cudaStreamDestroy(p->d2h);
  delete p;
}

int mxk_dit_block_ops_host(MxkHostPipeline* p, const MxkBlockArgs* a, int64_t* h2d_bytes,
                           int64_t* d2h_bytes) {
  if (!p) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_host: null pipeline");
  if (int rc = check_block(a)) return rc;
  if (a->dim != p->dim || a->F != p->F || a->H != p->H || a->D != p->D || a->rot != p->rot ||
      (a->v_in != nullptr) != (p->with_v != 0) || a->act_mode != p->act_mode)
    return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_host: args do not match the pipeline's shapes");
  if (a->rot > 0 && a->rope_mode != MXK_ROPE_NONE && (!a->cos || !a->sin))
    return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_host: rotary mode needs cos and sin");
  int64_t up = 0, down = 0;
  const int64_t dim = p->dim, inner = p->inner, F = p->F, half = p->half;
  const bool rope = a->rot > 0 && a->rope_mode != MXK_ROPE_NONE;
  cudaError_t e = cudaSuccess;
#define MXK_CU(call)                                                                              \
  do {                                                                                            \
    if ((e = (call)) != cudaSuccess) {                                                            \
      cudaStreamSynchronize(p->h2d), cudaStreamSynchronize(p->comp), cudaStreamSynchronize(p->d2h); \
      return fail(MXK_ERR_CUDA, "dit_block_ops_host: %s: %s", #call, cudaGetErrorString(e));      \
    }                                                                                             \
  } while (0)
  int64_t c = 0;
  for (int64_t r0 = 0; r0 < a->rows; r0 += p->chunk_rows, c++) {
    const int64_t n = a->rows - r0 < p->chunk_rows ? a->rows - r0 : p->chunk_rows;
    MxkHostPipeline::Slot& s = p->slot[c % kHostSlots];
    // upload (waits until the slot's previous results have left)
    if (c >= kHostSlots) MXK_CU(cudaStreamWaitEvent(p->h2d, s.d2h_done, 0));
    auto in = [&](void* dst, const void* src, int64_t bytes) {
      up += bytes;
      return cudaMemcpyAsync(dst, src, size_t(bytes), cudaMemcpyHostToDevice, p->h2d);
    };
    auto in2d = [&](mxk_bf16* dst, const mxk_bf16* src, int64_t col0) {
      // gather [n, inner] out of a strided host array into a dense staging array
      up += n * inner * 2;
      if (a->qkv_stride == inner)  // dense rows: one linear copy
        return cudaMemcpyAsync(dst, src + r0 * inner + col0, size_t(n * inner) * 2, cudaMemcpyHostToDevice, p->h2d);
      return cudaMemcpy2DAsync(dst, size_t(inner) * 2, src + r0 * a->qkv_stride + col0, size_t(a->qkv_stride) * 2,
                               size_t(inner) * 2, size_t(n), cudaMemcpyHostToDevice, p->h2d);
    };
    MXK_CU(in(s.x, a->x + r0 * dim, n * dim * 4));
    MXK_CU(in2d(s.q_in, a->q_in, a->q_col0));
    MXK_CU(in2d(s.k_in, a->k_in, a->k_col0));
    if (p->with_v) MXK_CU(in2d(s.v_in, a->v_in, a->v_col0));
    if (rope) {
      MXK_CU(in(s.cos, a->cos + r0 * half, n * half * 4));
      MXK_CU(in(s.sin, a->sin + r0 * half, n * half * 4));
    }
    MXK_CU(in(s.attn_o, a->attn_o + r0 * dim, n * dim * 2));
    if (p->act_mode == 0) MXK_CU(in(s.act, a->act + r0 * F, n * F * 2));
    else MXK_CU(in(s.act2, a->act2 + r0 * 2 * F, n * 2 * F * 2));
    MXK_CU(in(s.mlp_o, a->mlp_o + r0 * dim, n * dim * 2));
    MXK_CU(cudaEventRecord(s.h2d_done, p->h2d));

    // compute on the staged chunk
    MXK_CU(cudaStreamWaitEvent(p->comp, s.h2d_done, 0));
    MxkBlockArgs d = *a;
    d.rows = n, d.chunk_rows = 0;
    d.x = s.x, d.h1 = s.h1, d.h2 = s.h2, d.attn_o = s.attn_o, d.mlp_o = s.mlp_o, d.act = s.act, d.act2 = s.act2;
    d.q_in = s.q_in, d.k_in = s.k_in, d.v_in = p->with_v ? s.v_in : nullptr;
    d.qkv_stride = inner, d.q_col0 = d.k_col0 = d.v_col0 = 0;
    d.q_out = s.q_out, d.k_out = s.k_out, d.v_out = s.v_out;
    d.cos = rope ? s.cos : nullptr, d.sin = rope ? s.sin : nullptr;
    d.scale1 = shifted(a->scale1, r0), d.shift1 = shifted(a->shift1, r0), d.gate1 = shifted(a->gate1, r0);
    d.scale2 = shifted(a->scale2, r0), d.shift2 = shifted(a->shift2, r0), d.gate2 = shifted(a->gate2, r0);
    if (int rc = block_rows(d, 0, n, p->comp)) {
      cudaStreamSynchronize(p->h2d), cudaStreamSynchronize(p->comp), cudaStreamSynchronize(p->d2h);
      return rc;
    }
    MXK_CU(cudaEventRecord(s.comp_done, p->comp));

    // download
    MXK_CU(cudaStreamWaitEvent(p->d2h, s.comp_done, 0));
    auto outc = [&](void* dst, const void* src, int64_t bytes) {
      down += bytes;
      return cudaMemcpyAsync(dst, src, size_t(bytes), cudaMemcpyDeviceToHost, p->d2h);
    };
    MXK_CU(outc(a->h1 + r0 * dim, s.h1, n * dim * 2));
    MXK_CU(outc(a->q_out + r0 * inner, s.q_out, n * inner * 2));
    MXK_CU(outc(a->k_out + r0 * inner, s.k_out, n * inner * 2));
    if (p->with_v) MXK_CU(outc(a->v_out + r0 * inner, s.v_out, n * inner * 2));
    MXK_CU(outc(a->h2 + r0 * dim, s.h2, n * dim * 2));
    MXK_CU(outc(a->act + r0 * F, s.act, n * F * 2));
    MXK_CU(outc(a->x + r0 * dim, s.x, n * dim * 4));
    MXK_CU(cudaEventRecord(s.d2h_done, p->d2h));
  }
  MXK_CU(cudaStreamSynchronize(p->d2h));
#undef MXK_CU
  if (h2d_bytes) *h2d_bytes = up;
  if (d2h_bytes) *d2h_bytes = down;
  // the last download was ordered after every chunk's kernels, so the word is final by now
  return device_error_status("dit_block_ops_host", p->d2h);
}


// ---- block ops on host buffers without any allocation -------------------------------------------
//
// Staging for mxk_dit_block_ops_host_static.  The array lives in the library's device image: every
// GPU whose context loads libmxk holds these bytes until the process exits.  In host code the
// name g_static_stage is only a handle for the symbol - it is not a device address and must never
// be handed to a kernel or a copy; static_stage_base() asks the runtime for the real address.
constexpr size_t kStaticStageBytes = size_t(MXK_STATIC_STAGE_MIB) << 20;
static __device__ __align__(256) unsigned char g_static_stage[kStaticStageBytes];

namespace {
constexpr int kStaticMaxDevices = 64;
std::atomic<unsigned char*> g_static_base[kStaticMaxDevices];

// Device address of g_static_stage on the CURRENT device; looked up once per device (with that
// device current, as cudaGetSymbolAddress answers for the current device) and then cached.
int static_stage_base(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "dit_block_ops_host_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kStaticMaxDevices) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_host_static: device ordinal %d", dev);
  unsigned char* p = g_static_base[dev].load(std::memory_order_acquire);
  if (!p) {
    void* addr = nullptr;
    e = cudaGetSymbolAddress(&addr, g_static_stage);
    if (e != cudaSuccess || !addr)
      return fail(MXK_ERR_CUDA, "dit_block_ops_host_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    p = static_cast<unsigned char*>(addr);
    g_static_base[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return MXK_OK;
}
}  // namespace

int64_t mxk_static_stage_bytes(void) { return int64_t(kStaticStageBytes); }

int mxk_dit_block_ops_host_static(const MxkBlockArgs* a, mxk_stream_t stream, int64_t* h2d_bytes,
                                  int64_t* d2h_bytes) {
  if (int rc = check_block(a)) return rc;
  if (a->rot < 0 || a->rot > a->D) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_host_static: rot=%d", a->rot);
  const bool rope = a->rot > 0 && a->rope_mode != MXK_ROPE_NONE;
  if (rope && (!a->cos || !a->sin)) return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_host_static: rotary mode needs cos and sin");
  const bool with_v = a->v_in != nullptr;
  const int64_t dim = a->dim, inner = int64_t(a->H) * a->D, F = a->F, half = a->rot / 2;
  // bytes of staging one row needs, each array rounded up so that every array of a chunk starts on
  // a 256-byte boundary whatever the chunk's row count (the row count is kept a multiple of 64)
  auto pad = [](int64_t b) { return (b + 3) / 4 * 4; };  // per row: multiples of 4 bytes x 64 rows = 256
  const int64_t bx = pad(dim * 4), bh = pad(dim * 2), bi = pad(inner * 2), bf = pad(F * 2),
                bf2 = a->act_mode == 1 ? pad(2 * F * 2) : 0, bt = pad((half > 0 ? half : 1) * 4);
  const int64_t per_row = bx + 4 * bh + (with_v ? 6 : 4) * bi + bf + bf2 + 2 * bt;
  int64_t chunk = int64_t(kStaticStageBytes) / per_row / 64 * 64;
  if (chunk < 64)
    return fail(MXK_ERR_TOO_LARGE,
                "dit_block_ops_host_static: one row stages %lld bytes; 64 rows do not fit the %lld-byte static "
                "staging array (use mxk_dit_block_ops_host, whose pipeline allocates its own)",
                (long long)per_row, (long long)kStaticStageBytes);
  cudaStream_t s = as_stream(stream);
  // The array's address is looked up for the CURRENT device: a stream of another device would make the
  // copies below land in (or fail against) the wrong GPU's array half-way through the block.
  if (reinterpret_cast<uintptr_t>(s) > 2) {  // 0, 1 and 2 are the default-stream handles of the current device
    int cur = -1, sdev = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cudaStreamGetDevice(s, &sdev) == cudaSuccess) {
      if (cur != sdev)
        return fail(MXK_ERR_INVALID_ARG, "dit_block_ops_host_static: the stream belongs to device %d but device %d is "
                    "current; make the stream's device current before the call", sdev, cur);
    } else {
      cudaGetLastError();  // an unsupported query is not an error of this call
    }
  }
  unsigned char* base = nullptr;
  if (int rc = static_stage_base(&base)) return rc;

  unsigned char* c = base;
  auto take = [&](int64_t row_bytes) { unsigned char* r = c; c += row_bytes * chunk; return r; };
  float* sx = reinterpret_cast<float*>(take(bx));
  mxk_bf16* sh1 = reinterpret_cast<mxk_bf16*>(take(bh));
  mxk_bf16* sh2 = reinterpret_cast<mxk_bf16*>(take(bh));
  mxk_bf16* sattn = reinterpret_cast<mxk_bf16*>(take(bh));
  mxk_bf16* smlp = reinterpret_cast<mxk_bf16*>(take(bh));
  mxk_bf16* sq_in = reinterpret_cast<mxk_bf16*>(take(bi));
  mxk_bf16* sk_in = reinterpret_cast<mxk_bf16*>(take(bi));
  mxk_bf16* sq_out = reinterpret_cast<mxk_bf16*>(take(bi));
  mxk_bf16* sk_out = reinterpret_cast<mxk_bf16*>(take(bi));
  mxk_bf16* sv_in = with_v ? reinterpret_cast<mxk_bf16*>(take(bi)) : nullptr;
  mxk_bf16* sv_out = with_v ? reinterpret_cast<mxk_bf16*>(take(bi)) : nullptr;
  mxk_bf16* sact = reinterpret_cast<mxk_bf16*>(take(bf));
  mxk_bf16* sact2 = a->act_mode == 1 ? reinterpret_cast<mxk_bf16*>(take(bf2)) : nullptr;
  float* scos = reinterpret_cast<float*>(take(bt));
  float* ssin = reinterpret_cast<float*>(take(bt));

  int64_t up = 0, down = 0;
  cudaError_t e = cudaSuccess;
#define MXK_CU(call)                                                                                \
  do {                                                                                              \
    if ((e = (call)) != cudaSuccess) {                                                              \
      cudaStreamSynchronize(s);                                                                     \
      return fail(MXK_ERR_CUDA, "dit_block_ops_host_static: %s: %s", #call, cudaGetErrorString(e)); \
    }                                                                                               \
  } while (0)
  for (int64_t r0 = 0; r0 < a->rows; r0 += chunk) {
    const int64_t n = a->rows - r0 < chunk ? a->rows - r0 : chunk;
    auto in = [&](void* dst, const void* src, int64_t bytes) {
      up += bytes;
      return cudaMemcpyAsync(dst, src, size_t(bytes), cudaMemcpyHostToDevice, s);
    };
    auto in2d = [&](mxk_bf16* dst, const mxk_bf16* src, int64_t col0) {
      up += n * inner * 2;
      if (a->qkv_stride == inner)
        return cudaMemcpyAsync(dst, src + r0 * inner + col0, size_t(n * inner) * 2, cudaMemcpyHostToDevice, s);
      return cudaMemcpy2DAsync(dst, size_t(inner) * 2, src + r0 * a->qkv_stride + col0, size_t(a->qkv_stride) * 2,
                               size_t(inner) * 2, size_t(n), cudaMemcpyHostToDevice, s);
    };
    // Everything a kernel of this chunk reads is written first, by these copies or by an earlier
    // kernel of the chunk, so what the previous call left in the array is never seen and nothing
    // needs to be cleared.
    MXK_CU(in(sx, a->x + r0 * dim, n * dim * 4));
    MXK_CU(in2d(sq_in, a->q_in, a->q_col0));
    MXK_CU(in2d(sk_in, a->k_in, a->k_col0));
    if (with_v) MXK_CU(in2d(sv_in, a->v_in, a->v_col0));
    if (rope) {
      MXK_CU(in(scos, a->cos + r0 * half, n * half * 4));
      MXK_CU(in(ssin, a->sin + r0 * half, n * half * 4));
    }
    MXK_CU(in(sattn, a->attn_o + r0 * dim, n * dim * 2));
    if (a->act_mode == 0) MXK_CU(in(sact, a->act + r0 * F, n * F * 2));
    else MXK_CU(in(sact2, a->act2 + r0 * 2 * F, n * 2 * F * 2));
    MXK_CU(in(smlp, a->mlp_o + r0 * dim, n * dim * 2));

    MxkBlockArgs d = *a;
    d.rows = n, d.chunk_rows = 0;
    d.x = sx, d.h1 = sh1, d.h2 = sh2, d.attn_o = sattn, d.mlp_o = smlp, d.act = sact, d.act2 = sact2;
    d.q_in = sq_in, d.k_in = sk_in, d.v_in = sv_in;
    d.qkv_stride = inner, d.q_col0 = d.k_col0 = d.v_col0 = 0;
    d.q_out = sq_out, d.k_out = sk_out, d.v_out = sv_out;
    d.cos = rope ? scos : nullptr, d.sin = rope ? ssin : nullptr;
    d.scale1 = shifted(a->scale1, r0), d.shift1 = shifted(a->shift1, r0), d.gate1 = shifted(a->gate1, r0);
    d.scale2 = shifted(a->scale2, r0), d.shift2 = shifted(a->shift2, r0), d.gate2 = shifted(a->gate2, r0);
    if (int rc = block_rows(d, 0, n, stream)) {
      cudaStreamSynchronize(s);
      return rc;
    }

    auto outc = [&](void* dst, const void* src, int64_t bytes) {
      down += bytes;
      return cudaMemcpyAsync(dst, src, size_t(bytes), cudaMemcpyDeviceToHost, s);
    };
    MXK_CU(outc(a->h1 + r0 * dim, sh1, n * dim * 2));
    MXK_CU(outc(a->q_out + r0 * inner, sq_out, n * inner * 2));
    MXK_CU(outc(a->k_out + r0 * inner, sk_out, n * inner * 2));
    if (with_v) MXK_CU(outc(a->v_out + r0 * inner, sv_out, n * inner * 2));
    MXK_CU(outc(a->h2 + r0 * dim, sh2, n * dim * 2));
    MXK_CU(outc(a->act + r0 * F, sact, n * F * 2));
    MXK_CU(outc(a->x + r0 * dim, sx, n * dim * 4));
  }
#undef MXK_CU
  if (h2d_bytes) *h2d_bytes = up;
  if (d2h_bytes) *d2h_bytes = down;
  // one more 4-byte copy behind the last download (no allocation), then the wait for everything
  return device_error_status("dit_block_ops_host_static", s);
}

}  // extern "C"
