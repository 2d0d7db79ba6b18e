// head_norm_rope: per-head RMSNorm + rotary embedding + gather into [S, H, D]
// (reference: src/kernels/ops.cu:87-119 kernel, 197-210 launcher).
//
// For token s and head h:  v[d] = in[s*in_stride + col0 + h*D + d];  with norm_w:
// v = v * rsqrtf(mean_D(v^2) + eps) * norm_w[d];  for d < rot the value is rotated with its pair
// partner, (a, b) -> (a c - b s, a s + b c), pairs being (2i, 2i+1) in interleaved mode and
// (i, i + rot/2) in half mode, c/s = cos/sin[s*rot/2 + pair]; nothing is rounded between the
// norm and the rotation.
//
// Work layout of the fast kernel: a head is held by LPH = D/8 lanes, 8 consecutive channels
// (one 128-bit load) per lane.  A token is shared by `gpt` such lane groups; each group walks
// the heads gh, gh + gpt, ... of every tensor of the launch (q, k, v) with the token's cos/sin
// values in registers, so the table row is fetched once per token per group, not once per head.
#include "bulk_copy.cuh"
#include "common.cuh"
#include "tuning.h"

namespace mxk {
namespace {

constexpr int kMaxTensors = 3;
constexpr int kHeadsInFlight = 4;  // independent 128-bit loads each lane issues per batch
constexpr int kMaxScatterGroups = MXK_MAX_HEAD_GROUPS;

// What one bulk copy brings in: the bytes of one or more tensors for the tokens of a group.
struct CopySeg {
  const unsigned char* base;  // global address of token 0's first byte
  int64_t token_stride;       // bytes from one token to the next in global memory
  int token_bytes;            // bytes per token (multiple of 16)
  int smem_off;               // offset of the group's first token inside a stage
  int dense;                  // token_stride == token_bytes: a whole group is one contiguous copy
};

struct RopeArgs {
  MxkHeadTensor t[kMaxTensors];
  int n_tensors;
  int64_t S;
  int H, D;
  float eps;
  const float* cos;
  const float* sin;
  int gpt;              // lane groups per token
  int tokens_per_pass;  // tokens a CTA holds at once
  // bulk-copy pipeline kernel
  int passes, heads_per_pass, stages, stage_bytes;
  int rot, mode;    // shared by every rotating tensor of the launch
  int tpc;          // tokens per stage (one group)
  int64_t groups_per_cta;
  // interleaved assignment: `full_rounds` rounds in which CTA i takes group round * grid + i (tpc tokens each);
  // what is left (fewer than grid * tpc tokens, from tail_base on) is cut into one share of tail_tpc tokens per
  // CTA, so that the last round keeps every CTA busy on a smaller piece instead of a few CTAs on whole groups
  int full_rounds, tail_tpc;
  int64_t tail_base;
  int interleave;   // 1: CTA i takes groups i, i + grid, ...; 0: a contiguous range of groups
  // head-group scatter (register kernel only): head h of tensor ti goes to scatter_out[ti][h / heads_per_group]
  // at row scatter_row0 + s of a [*, heads_per_group, D] array (a peer GPU's buffer, or this GPU's own)
  int scatter_groups, heads_per_group;
  int64_t scatter_row0;
  mxk_bf16* scatter_out[kMaxTensors][kMaxScatterGroups];
  CopySeg seg[kMaxTensors];
  int n_seg;
  int t_seg[kMaxTensors];  // segment that holds tensor ti
  int t_off[kMaxTensors];  // byte offset of tensor ti's first head inside the token's segment bytes
  int cos_off, sin_off;    // table slots inside a stage
  int* err;
};

template <int LPH, bool SCATTER = false>
__global__ void __launch_bounds__(512) head_rope_kernel(const RopeArgs a) {
  constexpr int U = kHeadsInFlight;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int l = threadIdx.x % LPH;  // lane within the head: channels 8l .. 8l+7
  const int group = threadIdx.x / LPH;
  const int slot = group / a.gpt, gh = group % a.gpt;
  const bool slot_on = slot < a.tokens_per_pass;
  const int group_base = lane & ~(LPH - 1);
  const float inv_d = 1.f / float(a.D);
  (void)inv_d;

  for (int64_t s0 = int64_t(blockIdx.x) * a.tokens_per_pass; s0 < a.S;
       s0 += int64_t(gridDim.x) * a.tokens_per_pass) {
    const int64_t s = s0 + slot;
    const bool tok_on = slot_on && s < a.S;
    int cur_rot = -1, cur_mode = -1;
    float cs[8], sn[8];
    int partner = lane;
    bool rotates = false;
#pragma unroll 1
    for (int ti = 0; ti < a.n_tensors; ti++) {
      const MxkHeadTensor& t = a.t[ti];
      const int rot = t.mode == MXK_ROPE_NONE ? 0 : t.rot;
      if (rot != cur_rot || t.mode != cur_mode) {
        cur_rot = rot, cur_mode = t.mode;
        const int half = rot >> 1;
        rotates = 8 * l < rot;
        partner = lane;
        if (rotates && tok_on) {
          const float* cr = a.cos + s * half;
          const float* sr = a.sin + s * half;
          if (t.mode == MXK_ROPE_INTERLEAVED) {
            // channels 8l..8l+7 are pairs 4l..4l+3; even channels take -sin, odd ones +sin
            float4 c = *reinterpret_cast<const float4*>(cr + 4 * l);
            float4 q = *reinterpret_cast<const float4*>(sr + 4 * l);
            cs[0] = cs[1] = c.x, cs[2] = cs[3] = c.y, cs[4] = cs[5] = c.z, cs[6] = cs[7] = c.w;
            sn[0] = -q.x, sn[1] = q.x, sn[2] = -q.y, sn[3] = q.y;
            sn[4] = -q.z, sn[5] = q.z, sn[6] = -q.w, sn[7] = q.w;
          } else {
            const int hl = half >> 3;  // lanes per half
            const bool first = l < hl;
            const int lp = first ? l : l - hl;
            float4 c0 = *reinterpret_cast<const float4*>(cr + 8 * lp);
            float4 c1 = *reinterpret_cast<const float4*>(cr + 8 * lp + 4);
            float4 q0 = *reinterpret_cast<const float4*>(sr + 8 * lp);
            float4 q1 = *reinterpret_cast<const float4*>(sr + 8 * lp + 4);
            cs[0] = c0.x, cs[1] = c0.y, cs[2] = c0.z, cs[3] = c0.w;
            cs[4] = c1.x, cs[5] = c1.y, cs[6] = c1.z, cs[7] = c1.w;
            const float sg = first ? -1.f : 1.f;
            sn[0] = sg * q0.x, sn[1] = sg * q0.y, sn[2] = sg * q0.z, sn[3] = sg * q0.w;
            sn[4] = sg * q1.x, sn[5] = sg * q1.y, sn[6] = sg * q1.z, sn[7] = sg * q1.w;
          }
        }
        if (rotates && t.mode == MXK_ROPE_HALF) {
          const int hl = half >> 3;
          partner = group_base + (l < hl ? l + hl : l - hl);
        }
      }
      float w[8];
      if (t.norm_w) {
        float4 w0 = *reinterpret_cast<const float4*>(t.norm_w + 8 * l);
        float4 w1 = *reinterpret_cast<const float4*>(t.norm_w + 8 * l + 4);
        w[0] = w0.x, w[1] = w0.y, w[2] = w0.z, w[3] = w0.w;
        w[4] = w1.x, w[5] = w1.y, w[6] = w1.z, w[7] = w1.w;
      }
      const mxk_bf16* src = t.in + s * t.in_stride + t.col0 + 8 * l;
      mxk_bf16* dst = t.out + s * int64_t(a.H) * a.D + 8 * l;
      // Every lane of the CTA runs the same number of iterations (shuffles need whole warps).
      for (int h0 = 0; h0 < a.H; h0 += a.gpt * U) {
        uint4 raw[U];
        bool on[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int h = h0 + gh + u * a.gpt;
          on[u] = tok_on && h < a.H;
          raw[u] = make_uint4(0u, 0u, 0u, 0u);
          if (on[u]) raw[u] = ld_stream(reinterpret_cast<const uint4*>(src + int64_t(h) * a.D));
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          float v[8];
          unpack8(raw[u], v);
          if (t.norm_w) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) ss += v[i] * v[i];
            ss = group_sum<LPH>(ss);
            const float rstd = rsqrtf(ss / float(a.D) + a.eps);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = v[i] * rstd * w[i];
          }
          if (cur_mode == MXK_ROPE_INTERLEAVED) {
            if (rotates) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; i++) o[i] = v[i] * cs[i] + v[i ^ 1] * sn[i];
#pragma unroll
              for (int i = 0; i < 8; i++) v[i] = o[i];
            }
          } else if (cur_mode == MXK_ROPE_HALF && cur_rot > 0) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const float other = __shfl_sync(0xffffffffu, v[i], partner);
              if (rotates) v[i] = v[i] * cs[i] + other * sn[i];
            }
          }
          if (on[u]) {
            const int h = h0 + gh + u * a.gpt;
            if constexpr (SCATTER) {
              // the head's group decides the destination buffer; plain 128-bit stores, which reach a peer
              // GPU's memory over NVLink when the pointer is a peer mapping
              const int g = h / a.heads_per_group, hh = h - g * a.heads_per_group;
              mxk_bf16* o = a.scatter_out[ti][g] + ((a.scatter_row0 + s) * a.heads_per_group + hh) * int64_t(a.D) + 8 * l;
              *reinterpret_cast<uint4*>(o) = pack8(v);
            } else {
              st_stream(reinterpret_cast<uint4*>(dst + int64_t(h) * a.D), pack8(v));
            }
          }
        }
      }
    }
  }
}

// Bulk-copy (TMA) pipeline.  The last warp of the CTA is a producer: for each group of `tpc`
// consecutive tokens it issues cp.async.bulk copies of the tensors' bytes (one copy per group
// where the tokens are contiguous in memory, which is the case for a dense [S, H*D] projection
// and for a packed [S, 3*H*D] q|k|v buffer) and of the group's cos / sin rows into a
// shared-memory stage, completing on the stage's `full` mbarrier.  The other warps are consumers:
// thread t holds channels 8l..8l+7 (l = t % LPH) of head t / LPH (+ heads_per_pass per pass),
// reads them from the stage, normalises, rotates and stores 128 bits to global memory.  No warp
// depends on another one's heads, so there is no CTA-wide barrier in the loop: a warp that is
// done with a stage arrives on its `empty` mbarrier and the producer refills it once all have.
// Bytes in flight are stages x stage size per CTA, whatever the register count.
//
// All mbarrier waits are bounded (bulk_copy.cuh); a warp whose wait runs out records
// kErrBulkTimeout and leaves the loop, the others then run out too, and before the CTA exits the
// producer gives the copies it issued a bounded chance to land.
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Per-thread constants of a consumer: where its 8 channels sit and how they rotate.
struct LaneRole {
  int thread_off;   // byte offset of channels 8l..8l+7 of head hp inside a token's H*D bf16
  int pass_off;     // bytes from one pass's head to the next (heads_per_pass * D * 2)
  int tab_idx;      // first cos/sin entry of the lane (4 entries interleaved, 8 half mode)
  int partner;      // lane that holds the pair partners (half mode)
  int last_pass_heads;  // heads handled in the final pass (others handle heads_per_pass)
  int hp;
  bool rotates;     // 8l < rot
  bool first;       // half mode: the lane holds the first element of each pair
};

// All `ntok` tokens of one tensor inside a stage.  NORM: per-head RMSNorm; MODE as MXK_ROPE_*.
// src points at the thread's 8 channels of token 0 (pass 0) in shared memory, dst at the same
// place of the output; cr / sr at the lane's first table entry of token 0.
// PRELOAD (global-memory source, PASSES > 0): every pass's vector of a token is loaded before the first is used - the
// compiler cannot move a later pass's load above an earlier pass's store on its own (it cannot rule out that they alias).
template <int LPH, bool NORM, int MODE, int PASSES, bool PRELOAD = false>
__device__ __forceinline__ void rope_tokens(const unsigned char* src, int tok_bytes, const float* cr, const float* sr,
                                            int half, int ntok, unsigned char* dst, int out_tok_bytes,
                                            const float* w_row, float inv_d, float eps, int passes, int heads_per_pass,
                                            int H, const LaneRole& r) {
  float w[8];
  if (NORM) {
    const float4 w0 = *reinterpret_cast<const float4*>(w_row), w1 = *reinterpret_cast<const float4*>(w_row + 4);
    w[0] = w0.x, w[1] = w0.y, w[2] = w0.z, w[3] = w0.w, w[4] = w1.x, w[5] = w1.y, w[6] = w1.z, w[7] = w1.w;
  }
  for (int tk = 0; tk < ntok; tk++) {
    float c[8], sg[8];
    if (MODE == MXK_ROPE_INTERLEAVED) {
      // channels 8l..8l+7 are pairs 4l..4l+3: (a, b) -> (a c - b s, a s + b c)
      const float4 cc = *reinterpret_cast<const float4*>(cr), ss = *reinterpret_cast<const float4*>(sr);
      c[0] = cc.x, c[1] = cc.y, c[2] = cc.z, c[3] = cc.w;
      sg[0] = ss.x, sg[1] = ss.y, sg[2] = ss.z, sg[3] = ss.w;
    } else if (MODE == MXK_ROPE_HALF) {
      const float4 c0 = *reinterpret_cast<const float4*>(cr), c1 = *reinterpret_cast<const float4*>(cr + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sr), s1 = *reinterpret_cast<const float4*>(sr + 4);
      c[0] = c0.x, c[1] = c0.y, c[2] = c0.z, c[3] = c0.w, c[4] = c1.x, c[5] = c1.y, c[6] = c1.z, c[7] = c1.w;
      // the first element of a pair takes -sin, the second +sin
      const float f = r.first ? -1.f : 1.f;
      sg[0] = f * s0.x, sg[1] = f * s0.y, sg[2] = f * s0.z, sg[3] = f * s0.w;
      sg[4] = f * s1.x, sg[5] = f * s1.y, sg[6] = f * s1.z, sg[7] = f * s1.w;
    }
    const unsigned char* sp = src;
    unsigned char* dp = dst;
    uint4 pre[PRELOAD ? PASSES : 1];
    if (PRELOAD) {
#pragma unroll
      for (int pass = 0; pass < (PRELOAD ? PASSES : 0); pass++)
        pre[pass] = ld_stream(reinterpret_cast<const uint4*>(src + pass * r.pass_off));
    }
    // PASSES > 0: the pass count is a compile-time constant and every pass is full (H = PASSES *
    // heads_per_pass), so the loop unrolls into independent chains and needs no predicate.
#pragma unroll
    for (int pass = 0; pass < (PASSES > 0 ? PASSES : passes); pass++) {
      const bool on = PASSES > 0 || r.hp < (pass + 1 < passes ? heads_per_pass : H - pass * heads_per_pass);
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (PRELOAD) raw = pre[pass];
      else if (on) raw = *reinterpret_cast<const uint4*>(sp);
      float v[8];
      unpack8(raw, v);
      if (NORM) {
        float q = v[0] * v[0];
#pragma unroll
        for (int i = 1; i < 8; i++) q = fmaf(v[i], v[i], q);
        q = group_sum<LPH>(q);
        const float rstd = rsqrt_approx(fmaf(q, inv_d, eps));
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] * rstd * w[i];
      }
      if (MODE == MXK_ROPE_INTERLEAVED) {
        if (r.rotates) {
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const float a0 = v[2 * i], b0 = v[2 * i + 1];
            v[2 * i] = a0 * c[i] - b0 * sg[i];
            v[2 * i + 1] = b0 * c[i] + a0 * sg[i];
          }
        }
      } else if (MODE == MXK_ROPE_HALF) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float other = __shfl_sync(0xffffffffu, v[i], r.partner);
          if (r.rotates) v[i] = fmaf(other, sg[i], v[i] * c[i]);
        }
      }
      if (on) st_stream(reinterpret_cast<uint4*>(dp), pack8(v));
      sp += r.pass_off;
      dp += r.pass_off;
    }
    src += tok_bytes;
    dst += out_tok_bytes;
    cr += half;
    sr += half;
  }
}

// Sixteen channels per lane (the "wide" mapping): a head is held by LPH = D/16 lanes, lane l owning
// channels 8l..8l+7 (chunk A) and D/2 + 8l .. D/2 + 8l + 7 (chunk B).  Against the 8-channel mapping
// this halves the per-vector overhead (addressing, loop, barrier traffic), takes one shuffle round
// out of the head reduction and puts both elements of every half-mode pair (i, i + D/2) in the same
// lane, so that no partner exchange is needed when rot == D.
struct WideRole {
  int thread_off;  // byte offset of chunk A of head hp inside a token's H*D bf16
  int pass_off;    // bytes from one pass's head to the next
  int hp;
  int tab_a, tab_b;  // first cos/sin entry of chunk A / chunk B (interleaved), of the lane's 8 pairs (half: tab_a)
  bool rot_a, rot_b;  // the chunk lies inside the rotated channels
};

template <int LPH, bool NORM, int MODE, int PASSES>
__device__ __forceinline__ void rope_tokens_wide(const unsigned char* src, int tok_bytes, const float* cos_row, const float* sin_row,
                                                 int half, int ntok, unsigned char* dst, int out_tok_bytes, const float* w_a,
                                                 const float* w_b, int chunk_b_off, float inv_d, float eps, int passes,
                                                 int heads_per_pass, int H, const WideRole& r) {
  float wa[8], wb[8];
  if (NORM) {
    const float4 a0 = *reinterpret_cast<const float4*>(w_a), a1 = *reinterpret_cast<const float4*>(w_a + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(w_b), b1 = *reinterpret_cast<const float4*>(w_b + 4);
    wa[0] = a0.x, wa[1] = a0.y, wa[2] = a0.z, wa[3] = a0.w, wa[4] = a1.x, wa[5] = a1.y, wa[6] = a1.z, wa[7] = a1.w;
    wb[0] = b0.x, wb[1] = b0.y, wb[2] = b0.z, wb[3] = b0.w, wb[4] = b1.x, wb[5] = b1.y, wb[6] = b1.z, wb[7] = b1.w;
  }
  for (int tk = 0; tk < ntok; tk++) {
    // interleaved: c[0..3] / s[0..3] are chunk A's four pairs, c[4..7] / s[4..7] chunk B's;
    // half (rot == D): pair i of the lane is (A[i], B[i]) with table entry tab_a + i
    float c[8], sg[8];
    if (MODE == MXK_ROPE_INTERLEAVED) {
      const float4 ca = *reinterpret_cast<const float4*>(cos_row + r.tab_a), sa = *reinterpret_cast<const float4*>(sin_row + r.tab_a);
      c[0] = ca.x, c[1] = ca.y, c[2] = ca.z, c[3] = ca.w, sg[0] = sa.x, sg[1] = sa.y, sg[2] = sa.z, sg[3] = sa.w;
      if (r.rot_b) {
        const float4 cb = *reinterpret_cast<const float4*>(cos_row + r.tab_b), sb = *reinterpret_cast<const float4*>(sin_row + r.tab_b);
        c[4] = cb.x, c[5] = cb.y, c[6] = cb.z, c[7] = cb.w, sg[4] = sb.x, sg[5] = sb.y, sg[6] = sb.z, sg[7] = sb.w;
      } else {
        c[4] = c[5] = c[6] = c[7] = 1.f, sg[4] = sg[5] = sg[6] = sg[7] = 0.f;
      }
    } else if (MODE == MXK_ROPE_HALF) {
      const float4 c0 = *reinterpret_cast<const float4*>(cos_row + r.tab_a), c1 = *reinterpret_cast<const float4*>(cos_row + r.tab_a + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sin_row + r.tab_a), s1 = *reinterpret_cast<const float4*>(sin_row + r.tab_a + 4);
      c[0] = c0.x, c[1] = c0.y, c[2] = c0.z, c[3] = c0.w, c[4] = c1.x, c[5] = c1.y, c[6] = c1.z, c[7] = c1.w;
      sg[0] = s0.x, sg[1] = s0.y, sg[2] = s0.z, sg[3] = s0.w, sg[4] = s1.x, sg[5] = s1.y, sg[6] = s1.z, sg[7] = s1.w;
    }
    const unsigned char* sp = src;
    unsigned char* dp = dst;
#pragma unroll
    for (int pass = 0; pass < (PASSES > 0 ? PASSES : passes); pass++) {
      const bool on = PASSES > 0 || r.hp < (pass + 1 < passes ? heads_per_pass : H - pass * heads_per_pass);
      uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = make_uint4(0u, 0u, 0u, 0u);
      if (on) {
        ra = *reinterpret_cast<const uint4*>(sp);
        rb = *reinterpret_cast<const uint4*>(sp + chunk_b_off);
      }
      float va[8], vb[8];
      unpack8(ra, va);
      unpack8(rb, vb);
      if (NORM) {
        float qa = va[0] * va[0], qb = vb[0] * vb[0];
#pragma unroll
        for (int i = 1; i < 8; i++) qa = fmaf(va[i], va[i], qa), qb = fmaf(vb[i], vb[i], qb);
        const float q = group_sum<LPH>(qa + qb);
        const float rstd = rsqrt_approx(fmaf(q, inv_d, eps));
#pragma unroll
        for (int i = 0; i < 8; i++) va[i] = va[i] * rstd * wa[i], vb[i] = vb[i] * rstd * wb[i];
      }
      if (MODE == MXK_ROPE_INTERLEAVED) {
        if (r.rot_a) {
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const float a0 = va[2 * i], b0 = va[2 * i + 1];
            va[2 * i] = a0 * c[i] - b0 * sg[i];
            va[2 * i + 1] = b0 * c[i] + a0 * sg[i];
          }
        }
        if (r.rot_b) {
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const float a0 = vb[2 * i], b0 = vb[2 * i + 1];
            vb[2 * i] = a0 * c[4 + i] - b0 * sg[4 + i];
            vb[2 * i + 1] = b0 * c[4 + i] + a0 * sg[4 + i];
          }
        }
      } else if (MODE == MXK_ROPE_HALF) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float a0 = va[i], b0 = vb[i];
          va[i] = a0 * c[i] - b0 * sg[i];
          vb[i] = fmaf(a0, sg[i], b0 * c[i]);
        }
      }
      if (on) {
        st_stream(reinterpret_cast<uint4*>(dp), pack8(va));
        st_stream(reinterpret_cast<uint4*>(dp + chunk_b_off), pack8(vb));
      }
      sp += r.pass_off;
      dp += r.pass_off;
    }
    src += tok_bytes;
    dst += out_tok_bytes;
    cos_row += half;
    sin_row += half;
  }
}

// First token and token count of this CTA's it-th group.
__device__ __forceinline__ void rope_group(const RopeArgs& a, int it, int64_t g_begin, int64_t g_step, int64_t& s0, int& ntok) {
  if (a.interleave) {
    if (it < a.full_rounds) {
      s0 = (int64_t(it) * gridDim.x + blockIdx.x) * a.tpc;
      ntok = a.tpc;
    } else {
      s0 = a.tail_base + int64_t(blockIdx.x) * a.tail_tpc;
      ntok = int(a.S - s0 < a.tail_tpc ? a.S - s0 : a.tail_tpc);
    }
  } else {
    s0 = (g_begin + it * g_step) * a.tpc;
    ntok = int(a.S - s0 < a.tpc ? a.S - s0 : a.tpc);
  }
}

// The producer lane's loop: one group of `tpc` tokens per stage, in order; returns false when a
// bounded wait on an `empty` barrier ran out.  `issued` counts the groups whose copies went out.
__device__ __forceinline__ bool rope_produce(const RopeArgs& a, unsigned char* dyn, unsigned long long* full,
                                             unsigned long long* empty, int64_t g_begin, int64_t g_step, int it_begin, int it_end,
                                             int& issued) {
  const int half = a.rot >> 1;
  const bool rope = a.mode != MXK_ROPE_NONE && a.rot > 0;
  int st = 0;
  // Parity of the `empty` phase to wait for: the k-th refill of a stage (k >= 1) follows the
  // completion of its phase k - 1, so the first wait uses parity 0 and it flips per trip after that.
  unsigned ph = 0;
  for (int it = it_begin; it < it_end; it++) {
    if (it >= a.stages && !mbar_wait(smem_u32(&empty[st]), ph)) return false;
    int64_t s0;
    int ntok_i;
    rope_group(a, it, g_begin, g_step, s0, ntok_i);
    const unsigned ntok = unsigned(ntok_i);
    const unsigned bar = smem_u32(&full[st]);
    const unsigned dst = smem_u32(dyn + size_t(st) * a.stage_bytes);
    unsigned bytes = rope ? 2u * ntok * unsigned(half) * 4u : 0u;
    for (int i = 0; i < a.n_seg; i++) bytes += ntok * unsigned(a.seg[i].token_bytes);
    mbar_expect_tx(bar, bytes);
    for (int i = 0; i < a.n_seg; i++) {
      const CopySeg& sg = a.seg[i];
      const unsigned char* src = sg.base + s0 * sg.token_stride;
      if (sg.dense) {
        bulk_g2s(dst + sg.smem_off, src, ntok * unsigned(sg.token_bytes), bar);
      } else {
        for (unsigned t = 0; t < ntok; t++)
          bulk_g2s(dst + sg.smem_off + t * unsigned(sg.token_bytes), src + t * sg.token_stride, unsigned(sg.token_bytes), bar);
      }
    }
    if (rope) {
      bulk_g2s(dst + a.cos_off, a.cos + s0 * half, ntok * unsigned(half) * 4u, bar);
      bulk_g2s(dst + a.sin_off, a.sin + s0 * half, ntok * unsigned(half) * 4u, bar);
    }
    issued++;
    if (++st == a.stages) st = 0, ph ^= (it >= a.stages ? 1u : 0u);
  }
  return true;
}

// MINB (wide mapping only): 1 = CTAs of up to 128 threads, four per SM (at most 128 registers: one register more
// would cost the fourth CTA); 4 = CTAs of up to 160 threads, four per SM (96 registers); 0 = no promise.
template <int LPH, int PASSES = 0, bool WIDE = false, int MINB = 0>
__global__ void __launch_bounds__(!WIDE ? 544 : MINB == 1 ? 128 : 160, MINB == 0 ? 1 : 4) head_rope_pipe_kernel(const RopeArgs a) {
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ __align__(8) unsigned long long full[8], empty[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_cons_warps = (blockDim.x >> 5) - 1;
  const int half = a.rot >> 1;
  const bool rope = a.mode != MXK_ROPE_NONE && a.rot > 0;
  const int64_t n_groups = (a.S + a.tpc - 1) / a.tpc;
  // This CTA's groups: a contiguous range, or every gridDim.x-th group so that the grid sweeps one
  // compact window of tokens together.
  const int64_t g_step = a.interleave ? int64_t(gridDim.x) : 1;
  const int64_t g_begin = a.interleave ? int64_t(blockIdx.x) : int64_t(blockIdx.x) * a.groups_per_cta;
  const int64_t g_end = a.interleave ? n_groups : (g_begin + a.groups_per_cta < n_groups ? g_begin + a.groups_per_cta : n_groups);
  const int my_groups = a.interleave ? a.full_rounds + (a.tail_base + int64_t(blockIdx.x) * a.tail_tpc < a.S ? 1 : 0)
                                     : (g_end > g_begin ? int((g_end - g_begin + g_step - 1) / g_step) : 0);

  if (tid == 0) {
    for (int i = 0; i < a.stages; i++) {
      mbar_init(smem_u32(&full[i]), 1);
      mbar_init(smem_u32(&empty[i]), unsigned(n_cons_warps));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();
  __syncthreads();  // the barriers exist for every warp; still nothing has touched global memory
  pdl_wait();
  // No staging step between the dependency wait and the first copies: the producer issues at once, and the
  // consumers fetch their 8 (16) norm weights straight from global memory (L1 / L2 hits after the first stage)
  // while those copies are in flight.

  bool ok = true;
  int issued = 0;  // producer: groups whose copies were issued
  if (warp == n_cons_warps) {
    if (lane == 0) ok = rope_produce(a, dyn, full, empty, g_begin, g_step, 0, my_groups, issued);
  } else if constexpr (WIDE) {
    const int l = tid % LPH;
    WideRole r;
    r.hp = tid / LPH;
    r.thread_off = (r.hp * a.D + 8 * l) * 2;
    r.pass_off = a.heads_per_pass * a.D * 2;
    const int chunk_b_off = a.D;  // D/2 channels of bf16
    r.rot_a = rope && 8 * l < a.rot;
    r.rot_b = rope && a.D / 2 + 8 * l < a.rot;
    if (a.mode == MXK_ROPE_INTERLEAVED) {
      r.tab_a = r.rot_a ? 4 * l : 0;
      r.tab_b = r.rot_b ? a.D / 4 + 4 * l : 0;
    } else {
      r.tab_a = r.tab_b = 8 * l;  // half mode on this path has rot == D: pair i of the lane is entry 8l + i
    }
    const float inv_d = 1.f / float(a.D);
    const int tok_out_bytes = a.H * a.D * 2;
    int st = 0;
    unsigned ph = 0;
    for (int it = 0; it < my_groups; it++) {
      if (!mbar_wait(smem_u32(&full[st]), ph)) {
        ok = false;
        break;
      }
      const unsigned char* stage = dyn + size_t(st) * a.stage_bytes;
      int64_t s0;
      int ntok;
      rope_group(a, it, g_begin, g_step, s0, ntok);
      const float* cr = reinterpret_cast<const float*>(stage + a.cos_off);
      const float* sr = reinterpret_cast<const float*>(stage + a.sin_off);
#pragma unroll 1
      for (int ti = 0; ti < a.n_tensors; ti++) {
        const MxkHeadTensor& t = a.t[ti];
        const CopySeg& sg = a.seg[a.t_seg[ti]];
        const unsigned char* src = stage + sg.smem_off + a.t_off[ti] + r.thread_off;
        unsigned char* dst = reinterpret_cast<unsigned char*>(t.out) + s0 * tok_out_bytes + r.thread_off;
        const bool t_rope = t.mode != MXK_ROPE_NONE && t.rot > 0;
        const float* wa = t.norm_w ? t.norm_w + 8 * l : nullptr;
        const float* wb = t.norm_w ? t.norm_w + a.D / 2 + 8 * l : nullptr;
#define MXK_ROPE_CALL(NORM, MODE)                                                                                      \
  rope_tokens_wide<LPH, NORM, MODE, PASSES>(src, sg.token_bytes, cr, sr, half, ntok, dst, tok_out_bytes, wa, wb, chunk_b_off, \
                                            inv_d, a.eps, a.passes, a.heads_per_pass, a.H, r)
        if (t.norm_w) {
          if (!t_rope) MXK_ROPE_CALL(true, MXK_ROPE_NONE);
          else if (a.mode == MXK_ROPE_INTERLEAVED) MXK_ROPE_CALL(true, MXK_ROPE_INTERLEAVED);
          else MXK_ROPE_CALL(true, MXK_ROPE_HALF);
        } else {
          if (!t_rope) MXK_ROPE_CALL(false, MXK_ROPE_NONE);
          else if (a.mode == MXK_ROPE_INTERLEAVED) MXK_ROPE_CALL(false, MXK_ROPE_INTERLEAVED);
          else MXK_ROPE_CALL(false, MXK_ROPE_HALF);
        }
#undef MXK_ROPE_CALL
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty[st]));
      if (++st == a.stages) st = 0, ph ^= 1u;
    }
  } else {
    const int l = tid % LPH;
    LaneRole r;
    r.hp = tid / LPH;
    r.thread_off = (r.hp * a.D + 8 * l) * 2;
    r.pass_off = a.heads_per_pass * a.D * 2;
    r.rotates = rope && 8 * l < a.rot;
    r.tab_idx = 0, r.partner = lane, r.first = true;
    if (r.rotates) {
      if (a.mode == MXK_ROPE_INTERLEAVED) {
        r.tab_idx = 4 * l;
      } else {
        const int hl = half >> 3;
        r.first = l < hl;
        r.tab_idx = 8 * (r.first ? l : l - hl);
        r.partner = (lane & ~(LPH - 1)) + (r.first ? l + hl : l - hl);
      }
    }
    const float inv_d = 1.f / float(a.D);  // D is a power of two on this path: exact
    const int tok_out_bytes = a.H * a.D * 2;

    int st = 0;
    unsigned ph = 0;
    for (int it = 0; it < my_groups; it++) {
      if (!mbar_wait(smem_u32(&full[st]), ph)) {
        ok = false;
        break;
      }
      const unsigned char* stage = dyn + size_t(st) * a.stage_bytes;
      int64_t s0;
      int ntok;
      rope_group(a, it, g_begin, g_step, s0, ntok);
      const float* cr = reinterpret_cast<const float*>(stage + a.cos_off) + r.tab_idx;
      const float* sr = reinterpret_cast<const float*>(stage + a.sin_off) + r.tab_idx;
#pragma unroll 1
      for (int ti = 0; ti < a.n_tensors; ti++) {
        {
          const MxkHeadTensor& t = a.t[ti];
          const CopySeg& sg = a.seg[a.t_seg[ti]];
          const unsigned char* src = stage + sg.smem_off + a.t_off[ti] + r.thread_off;
          unsigned char* dst = reinterpret_cast<unsigned char*>(t.out) + s0 * tok_out_bytes + r.thread_off;
          const bool t_rope = t.mode != MXK_ROPE_NONE && t.rot > 0;
          const float* wr = t.norm_w ? t.norm_w + 8 * l : nullptr;
#define MXK_ROPE_CALL(NORM, MODE)                                                                          \
  rope_tokens<LPH, NORM, MODE, PASSES>(src, sg.token_bytes, cr, sr, half, ntok, dst, tok_out_bytes, wr, inv_d, a.eps, \
                               a.passes, a.heads_per_pass, a.H, r)
          if (t.norm_w) {
            if (!t_rope) MXK_ROPE_CALL(true, MXK_ROPE_NONE);
            else if (a.mode == MXK_ROPE_INTERLEAVED) MXK_ROPE_CALL(true, MXK_ROPE_INTERLEAVED);
            else MXK_ROPE_CALL(true, MXK_ROPE_HALF);
          } else {
            if (!t_rope) MXK_ROPE_CALL(false, MXK_ROPE_NONE);
            else if (a.mode == MXK_ROPE_INTERLEAVED) MXK_ROPE_CALL(false, MXK_ROPE_INTERLEAVED);
            else MXK_ROPE_CALL(false, MXK_ROPE_HALF);
          }
#undef MXK_ROPE_CALL
        }
      }
      // The stage's bytes are in this warp's registers (they fed the stores above): hand it back.
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty[st]));
      if (++st == a.stages) st = 0, ph ^= 1u;
    }
  }

  if (!ok && a.err) atomicExch(a.err, kErrBulkTimeout);
  // Every warp reaches this barrier (all waits above are bounded).  On the normal path every
  // issued copy has been consumed, hence completed; after a failure the producer waits, bounded,
  // for the copies of its last `stages` groups so that none lands in a dead CTA's shared memory.
  const bool any_failed = __syncthreads_or(!ok) != 0;
  if (any_failed && warp == n_cons_warps && lane == 0) {
    for (int it = issued > a.stages ? issued - a.stages : 0; it < issued; it++)
      mbar_wait(smem_u32(&full[it % a.stages]), unsigned((it / a.stages) & 1));
  }
}

// The consumers' arithmetic of the pipeline straight from global memory, ONE group of tokens per CTA and as many CTAs
// as that takes (rope_path = 3): thread layout, passes and roles as in head_rope_pipe_kernel, no stages, no producer.
template <int LPH, int PASSES>
__global__ void __launch_bounds__(256) head_rope_tile_kernel(const RopeArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31;
  const int half = a.rot >> 1;
  const bool rope = a.mode != MXK_ROPE_NONE && a.rot > 0;
  const int l = tid % LPH;
  LaneRole r;
  r.hp = tid / LPH;
  r.thread_off = (r.hp * a.D + 8 * l) * 2;
  r.pass_off = a.heads_per_pass * a.D * 2;
  r.rotates = rope && 8 * l < a.rot;
  r.tab_idx = 0, r.partner = lane, r.first = true;
  if (r.rotates) {
    if (a.mode == MXK_ROPE_INTERLEAVED) {
      r.tab_idx = 4 * l;
    } else {
      const int hl = half >> 3;
      r.first = l < hl;
      r.tab_idx = 8 * (r.first ? l : l - hl);
      r.partner = (lane & ~(LPH - 1)) + (r.first ? l + hl : l - hl);
    }
  }
  const float inv_d = 1.f / float(a.D);
  const int tok_out_bytes = a.H * a.D * 2;
  const int64_t s0 = int64_t(blockIdx.x) * a.tpc;
  const int ntok = int(a.S - s0 < a.tpc ? a.S - s0 : a.tpc);
  const float* cr = rope ? a.cos + s0 * half + r.tab_idx : nullptr;
  const float* sr = rope ? a.sin + s0 * half + r.tab_idx : nullptr;
#pragma unroll 1
  for (int ti = 0; ti < a.n_tensors; ti++) {
    const MxkHeadTensor& t = a.t[ti];
    const unsigned char* src = reinterpret_cast<const unsigned char*>(t.in + s0 * t.in_stride + t.col0) + r.thread_off;
    unsigned char* dst = reinterpret_cast<unsigned char*>(t.out) + s0 * tok_out_bytes + r.thread_off;
    const int tok_bytes = int(t.in_stride * 2);
    const bool t_rope = t.mode != MXK_ROPE_NONE && t.rot > 0;
    const float* wr = t.norm_w ? t.norm_w + 8 * l : nullptr;
#define MXK_ROPE_CALL(NORM, MODE)                                                                                        \
  rope_tokens<LPH, NORM, MODE, PASSES, (PASSES > 0)>(src, tok_bytes, cr, sr, half, ntok, dst, tok_out_bytes, wr, inv_d, a.eps, \
                                                     a.passes, a.heads_per_pass, a.H, r)
    if (t.norm_w) {
      if (!t_rope) MXK_ROPE_CALL(true, MXK_ROPE_NONE);
      else if (a.mode == MXK_ROPE_INTERLEAVED) MXK_ROPE_CALL(true, MXK_ROPE_INTERLEAVED);
      else MXK_ROPE_CALL(true, MXK_ROPE_HALF);
    } else {
      if (!t_rope) MXK_ROPE_CALL(false, MXK_ROPE_NONE);
      else if (a.mode == MXK_ROPE_INTERLEAVED) MXK_ROPE_CALL(false, MXK_ROPE_INTERLEAVED);
      else MXK_ROPE_CALL(false, MXK_ROPE_HALF);
    }
#undef MXK_ROPE_CALL
  }
}

// Any even D <= 256, any rot, any alignment: one warp per (token, head), the head's values pass
// through shared memory for the partner exchange.
__global__ void __launch_bounds__(256) head_rope_generic_kernel(const RopeArgs a) {
  __shared__ float buf[8][256];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float* hv = buf[wid];
  const int64_t total = a.S * a.H;
  for (int64_t item = int64_t(blockIdx.x) * 8 + wid; item < total; item += int64_t(gridDim.x) * 8) {
    const int64_t s = item / a.H;
    const int h = int(item % a.H);
    for (int ti = 0; ti < a.n_tensors; ti++) {
      const MxkHeadTensor& t = a.t[ti];
      const bf16* src = reinterpret_cast<const bf16*>(t.in) + s * t.in_stride + t.col0 + int64_t(h) * a.D;
      bf16* dst = reinterpret_cast<bf16*>(t.out) + (s * a.H + h) * a.D;
      float ss = 0.f;
      for (int d = lane; d < a.D; d += 32) {
        float v = bf16_to_f(src[d]);
        hv[d] = v;
        ss += v * v;
      }
      if (t.norm_w) {
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / float(a.D) + a.eps);
        for (int d = lane; d < a.D; d += 32) hv[d] = hv[d] * rstd * t.norm_w[d];
      }
      __syncwarp();
      const int rot = t.mode == MXK_ROPE_NONE ? 0 : t.rot, half = rot >> 1;
      for (int d = lane; d < a.D; d += 32) {
        float v = hv[d];
        if (d < rot) {
          int pair, idx;
          float other;
          if (t.mode == MXK_ROPE_INTERLEAVED) {
            pair = d >> 1, idx = d & 1, other = hv[d ^ 1];
          } else {
            pair = d < half ? d : d - half, idx = d < half ? 0 : 1;
            other = hv[d < half ? d + half : d - half];
          }
          const float c = a.cos[s * half + pair], si = a.sin[s * half + pair];
          v = idx == 0 ? v * c - other * si : other * si + v * c;
        }
        dst[d] = __float2bfloat16(v);
      }
      __syncwarp();
    }
  }
}

bool fast_ok(const RopeArgs& a) {
  const int D = a.D;
  if (!(D == 32 || D == 64 || D == 128 || D == 256)) return false;
  bool any_rot = false;
  for (int i = 0; i < a.n_tensors; i++) {
    const MxkHeadTensor& t = a.t[i];
    if (!aligned(t.in, 16) || !aligned(t.out, 16) || t.in_stride % 8 || t.col0 % 8) return false;
    if (t.norm_w && !aligned(t.norm_w, 16)) return false;
    if (t.mode == MXK_ROPE_INTERLEAVED && t.rot % 8) return false;
    if (t.mode == MXK_ROPE_HALF && t.rot % 16) return false;
    if (t.mode != MXK_ROPE_NONE && t.rot > 0) any_rot = true;
  }
  if (any_rot && (!aligned(a.cos, 16) || !aligned(a.sin, 16))) return false;
  return true;
}

// Plans the bulk-copy pipeline: beyond fast_ok it needs one (rot, mode) for all rotating tensors
// and table rows that are multiples of 16 bytes.  Tensors that are consecutive column blocks of
// the same buffer (packed q|k|v) become one copy segment.
bool pipe_plan(RopeArgs& a, bool wide = false) {
  a.rot = 0, a.mode = MXK_ROPE_NONE;
  for (int i = 0; i < a.n_tensors; i++) {
    const MxkHeadTensor& t = a.t[i];
    if (t.mode == MXK_ROPE_NONE || t.rot == 0) continue;
    if (a.mode == MXK_ROPE_NONE) a.rot = t.rot, a.mode = t.mode;
    else if (a.rot != t.rot || a.mode != t.mode) return false;
  }
  const int half = a.rot / 2;
  if (a.mode != MXK_ROPE_NONE && half % 4) return false;
  // the wide mapping needs a 32-byte head half and, in half mode, both elements of a pair in one lane (rot == D)
  if (wide && (a.D % 16 != 0 || (a.mode == MXK_ROPE_HALF && a.rot != a.D))) return false;
  const int lph = wide ? a.D / 16 : a.D / 8;
  int max_threads = tune(TUNE_ROPE_THREADS, 128);  // small CTAs, many per SM: measured best on B200
  if (max_threads > 512) max_threads = 512;
  if (max_threads < lph) max_threads = lph;
  int passes = 1;
  while (lph * int(ceil_div(a.H, passes)) > max_threads) passes++;
  if (wide) {
    // prefer a pass count that divides H into full warps (the pass loop then unrolls without predicates)
    for (int p = passes; p <= passes + 6 && p <= a.H; p++)
      if (a.H % p == 0 && (lph * (a.H / p)) % 32 == 0) {
        passes = p;
        break;
      }
  }
  a.passes = passes;
  a.heads_per_pass = int(ceil_div(a.H, passes));
  const int64_t hd = int64_t(a.H) * a.D;
  if (hd * 2 > (1 << 20)) return false;

  // one segment when the tensors are adjacent column blocks of one buffer, in order
  bool packed = a.n_tensors > 1;
  for (int i = 1; i < a.n_tensors && packed; i++)
    packed = a.t[i].in == a.t[0].in && a.t[i].in_stride == a.t[0].in_stride && a.t[i].col0 == a.t[0].col0 + i * hd;
  a.n_seg = packed ? 1 : a.n_tensors;
  for (int i = 0; i < a.n_seg; i++) {
    CopySeg& sg = a.seg[i];
    const MxkHeadTensor& t = a.t[i];
    sg.base = reinterpret_cast<const unsigned char*>(t.in + t.col0);
    sg.token_stride = t.in_stride * 2;
    sg.token_bytes = int((packed ? a.n_tensors * hd : hd) * 2);
    sg.dense = sg.token_stride == sg.token_bytes;
  }
  for (int i = 0; i < a.n_tensors; i++) {
    a.t_seg[i] = packed ? 0 : i;
    a.t_off[i] = packed ? int(i * hd * 2) : 0;
  }
  int per_token = 2 * half * 4;
  for (int i = 0; i < a.n_seg; i++) per_token += a.seg[i].token_bytes;
  int tpc = tune(TUNE_ROPE_TOKENS, 0);
  if (tpc <= 0) tpc = 16384 / per_token;
  if (tpc < 1) tpc = 1;
  if (tpc > 16) tpc = 16;
  a.tpc = tpc;
  int off = 0;
  for (int i = 0; i < a.n_seg; i++) {
    a.seg[i].smem_off = off;
    off += (tpc * a.seg[i].token_bytes + 127) & ~127;
  }
  a.cos_off = off;
  off += (tpc * half * 4 + 127) & ~127;
  a.sin_off = off;
  off += (tpc * half * 4 + 127) & ~127;
  a.stage_bytes = off;
  int stages = tune(TUNE_ROPE_STAGES, 0);
  if (stages <= 0) stages = 2;
  if (stages < 2) stages = 2;
  if (stages > 8) stages = 8;
  a.stages = stages;
  return size_t(stages) * a.stage_bytes <= 200 * 1024;
}

template <int LPH, int PASSES = 0, bool WIDE = false, int MINB = 0>
int launch_pipe(const char* name, RopeArgs a, cudaStream_t stream) {
  auto k = head_rope_pipe_kernel<LPH, PASSES, WIDE, MINB>;
  const int threads = int(ceil_div(int64_t(LPH) * a.heads_per_pass, 32) * 32) + 32;  // consumers + producer warp
  const size_t smem = size_t(a.stages) * a.stage_bytes;
  if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  const int per_sm = tune(TUNE_ROPE_CTAS_PER_SM, resident_ctas(k, threads, smem));
  const int64_t n_groups = ceil_div(a.S, a.tpc);
  int64_t ctas = int64_t(sm_count()) * (per_sm > 0 ? per_sm : 1);
  if (ctas > n_groups) ctas = n_groups;
  a.groups_per_cta = ceil_div(n_groups, ctas);
  a.interleave = tune(TUNE_PIPE_INTERLEAVE, 1) == 1;
  a.err = device_error_word();
  const int64_t grid = ceil_div(n_groups, a.groups_per_cta);
  a.full_rounds = int(a.S / (grid * a.tpc));
  a.tail_base = int64_t(a.full_rounds) * grid * a.tpc;
  a.tail_tpc = int(ceil_div(a.S - a.tail_base, grid));  // 0 when the rounds cover every token
  launch_pdl(k, dim3(unsigned(grid)), dim3(threads), smem, stream, a);
  return after_launch(name);
}

template <bool SCATTER>
int launch_register(const char* name, RopeArgs a, cudaStream_t stream);
int launch_generic(const char* name, RopeArgs a, cudaStream_t stream);

template <int PASSES>
int launch_tile(const char* name, RopeArgs a, cudaStream_t stream) {
  int tpc = tune(TUNE_ROPE_TOKENS, 1);
  if (tpc < 1) tpc = 1;
  a.tpc = tpc;
  const int threads = 16 * a.heads_per_pass;
  launch_pdl(head_rope_tile_kernel<16, PASSES>, dim3(unsigned(ceil_div(a.S, tpc))), dim3(threads), 0, stream, a);
  return after_launch(name);
}

int run(const char* name, RopeArgs a, cudaStream_t stream) {
  // D = 128 (every model shape): sixteen channels per lane, eight lanes per head
  // (opt-in, rope_wide = 1: measured within 2 % of the eight-channel mapping on every model shape, so the mapping with
  // the lower register count stays the default)
  if (a.D == 128 && fast_ok(a) && tune(TUNE_ROPE_PATH, 1) == 1 && tune(TUNE_ROPE_WIDE, 2) == 1 && a.S >= 2 && pipe_plan(a, true)) {
    const bool exact = a.H == a.passes * a.heads_per_pass && (8 * a.heads_per_pass) % 32 == 0;
    if (exact && tune(TUNE_ROPE_UNROLL, 1) == 1 && 8 * a.heads_per_pass + 32 <= 160) {
      // register budget of the unrolled kernel: CTAs of at most 128 threads are held to 128 registers (four CTAs
      // per SM), larger ones (32 heads: 160 threads) to 96; rope_wide_regs = 2 asks for 96 everywhere
      const bool small = 8 * a.heads_per_pass + 32 <= 128 && tune(TUNE_ROPE_WIDE_REGS, 1) == 1;
#define MXK_WIDE_CASE(P) \
  case P:                \
    return small ? launch_pipe<8, P, true, 1>(name, a, stream) : launch_pipe<8, P, true, 4>(name, a, stream)
      switch (a.passes) {
        MXK_WIDE_CASE(1);
        MXK_WIDE_CASE(2);
        MXK_WIDE_CASE(3);
        MXK_WIDE_CASE(4);
        MXK_WIDE_CASE(5);
        MXK_WIDE_CASE(7);
        default: break;
      }
#undef MXK_WIDE_CASE
    }
    if (8 * a.heads_per_pass + 32 <= 160) return launch_pipe<8, 0, true>(name, a, stream);
  }
  // a single tensor without norm and rotation is a strided copy: that one is faster in the tile form also as the default
  // (33272 tokens x 40 heads out of a packed q | k | v buffer: 102 us against 118 us through the pipeline)
  const bool copy_only = a.n_tensors == 1 && !a.t[0].norm_w && (a.t[0].mode == MXK_ROPE_NONE || a.t[0].rot == 0);
  const int rope_path = tune(TUNE_ROPE_PATH, copy_only ? 3 : 1);
  if (a.D == 128 && fast_ok(a) && rope_path == 3 && a.S < (int64_t(1) << 31) && pipe_plan(a) &&
      16 * a.heads_per_pass <= 256 && (16 * a.heads_per_pass) % 32 == 0) {
    const bool exact = a.H == a.passes * a.heads_per_pass;
    if (exact) {
      switch (a.passes) {
        case 3: return launch_tile<3>(name, a, stream);
        case 4: return launch_tile<4>(name, a, stream);
        case 5: return launch_tile<5>(name, a, stream);
        case 7: return launch_tile<7>(name, a, stream);
        default: break;
      }
    }
    return launch_tile<0>(name, a, stream);
  }
  if (fast_ok(a) && tune(TUNE_ROPE_PATH, 1) == 1 && a.S >= 2 && pipe_plan(a)) {
    switch (a.D / 8) {
      case 4: return launch_pipe<4>(name, a, stream);
      case 8: return launch_pipe<8>(name, a, stream);
      case 16: {
        // D = 128, the model shapes: when every pass is full and every consumer thread has a head, the
        // pass loop is unrolled at compile time (24, 32, 40, 56 heads at 8 heads per pass)
        const bool exact = a.H == a.passes * a.heads_per_pass && (16 * a.heads_per_pass) % 32 == 0;
        if (exact && tune(TUNE_ROPE_UNROLL, 1) == 1) {
          switch (a.passes) {
            case 3: return launch_pipe<16, 3>(name, a, stream);
            case 4: return launch_pipe<16, 4>(name, a, stream);
            case 5: return launch_pipe<16, 5>(name, a, stream);
            case 7: return launch_pipe<16, 7>(name, a, stream);
            default: break;
          }
        }
        return launch_pipe<16>(name, a, stream);
      }
      default: return launch_pipe<32>(name, a, stream);
    }
  }
  if (fast_ok(a)) return launch_register<false>(name, a, stream);
  return launch_generic(name, a, stream);
}

template <bool SCATTER>
int launch_register(const char* name, RopeArgs a, cudaStream_t stream) {
  {
    const int lph = a.D / 8;
    a.gpt = int(ceil_div(a.H, kHeadsInFlight));
    const int per_token = lph * a.gpt;
    if (per_token <= 512) {
      const int want = tune(TUNE_ROPE_THREADS, 256);
      int tpp = want / per_token;
      if (tpp < 1) tpp = 1;
      int threads = int(ceil_div(int64_t(per_token) * tpp, 32) * 32);
      a.tokens_per_pass = tpp;
      auto go = [&](auto kern) {
        // The scatter form (stores that cross NVLink) runs one group of tokens per CTA, as many CTAs as that takes:
        // 369 us against 418 us for one resident wave on 16636 tokens x 3 x 40 heads at two GPUs (0.90 against 0.80 of
        // the peer-copy rate).  The local form keeps the resident wave (31 us against 34 us on 8704 x 24 heads).
        const int per_sm = tune(TUNE_ROPE_CTAS_PER_SM, SCATTER ? (1 << 20) : resident_ctas(kern, threads));
        int64_t grid = ceil_div(a.S, tpp);
        const int64_t cap = int64_t(sm_count()) * (per_sm > 0 ? per_sm : 1);
        if (grid > cap) grid = cap;
        launch_pdl(kern, dim3(unsigned(grid)), dim3(threads), 0, stream, a);
      };
      switch (lph) {
        case 4: go(head_rope_kernel<4, SCATTER>); break;
        case 8: go(head_rope_kernel<8, SCATTER>); break;
        case 16: go(head_rope_kernel<16, SCATTER>); break;
        default: go(head_rope_kernel<32, SCATTER>); break;
      }
      return after_launch(name);
    }
  }
  if (SCATTER) return fail(MXK_ERR_INVALID_ARG, "%s: H * D / 8 = %d lanes per token exceed a CTA", name, a.D / 8 * a.gpt);
  return launch_generic(name, a, stream);
}

int launch_generic(const char* name, RopeArgs a, cudaStream_t stream) {
  int64_t grid = ceil_div(a.S * a.H, 8);
  const int64_t cap = int64_t(sm_count()) * 32;
  if (grid > cap) grid = cap;
  head_rope_generic_kernel<<<unsigned(grid), 256, 0, stream>>>(a);
  return after_launch(name);
}

int check(const char* name, const MxkHeadTensor& t, int H, int D, const float* cos, const float* sin) {
  if (!t.in || !t.out) return fail(MXK_ERR_INVALID_ARG, "%s: null in or out", name);
  if (t.mode != MXK_ROPE_NONE && t.mode != MXK_ROPE_INTERLEAVED && t.mode != MXK_ROPE_HALF)
    return fail(MXK_ERR_INVALID_ARG, "%s: unknown rope mode %d", name, t.mode);
  // the reference's own argument check (src/kernels/ops.cu:201)
  if (!(D > 0 && D % 2 == 0 && D <= 256 && t.rot >= 0 && t.rot <= D && t.rot % 2 == 0))
    return fail(MXK_ERR_INVALID_ARG, "%s: D=%d rot=%d", name, D, t.rot);
  if (H <= 0) return fail(MXK_ERR_INVALID_ARG, "%s: H=%d", name, H);
  if (t.in_stride < 0 || t.col0 < 0) return fail(MXK_ERR_INVALID_ARG, "%s: negative in_stride or col0", name);
  if (t.mode != MXK_ROPE_NONE && t.rot > 0 && (!cos || !sin))
    return fail(MXK_ERR_INVALID_ARG, "%s: rotary mode %d needs cos and sin tables", name, t.mode);
  return MXK_OK;
}

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int mxk_head_norm_rope(const mxk_bf16* in, int64_t S, int64_t in_stride, int64_t col0, int H,
                       int D, const float* norm_w, float eps, const float* cos, const float* sin,
                       int rot, int mode, mxk_bf16* out, mxk_stream_t stream) {
  if (S <= 0) return MXK_OK;
  RopeArgs a{};
  a.t[0] = MxkHeadTensor{in, in_stride, col0, norm_w, out, rot, mode};
  a.n_tensors = 1;
  a.S = S, a.H = H, a.D = D, a.eps = eps, a.cos = cos, a.sin = sin;
  if (int rc = check("head_norm_rope", a.t[0], H, D, cos, sin)) return rc;
  return run("head_norm_rope", a, as_stream(stream));
}

int mxk_qkv_norm_rope(const MxkHeadTensor* tensors_host, int n_tensors, int64_t S, int H, int D,
                      float eps, const float* cos, const float* sin, mxk_stream_t stream) {
  if (S <= 0 || n_tensors == 0) return MXK_OK;
  if (!tensors_host || n_tensors < 0 || n_tensors > kMaxTensors)
    return fail(MXK_ERR_INVALID_ARG, "qkv_norm_rope: n_tensors=%d (1..%d)", n_tensors, kMaxTensors);
  RopeArgs a{};
  for (int i = 0; i < n_tensors; i++) {
    a.t[i] = tensors_host[i];
    if (int rc = check("qkv_norm_rope", a.t[i], H, D, cos, sin)) return rc;
  }
  a.n_tensors = n_tensors;
  a.S = S, a.H = H, a.D = D, a.eps = eps, a.cos = cos, a.sin = sin;
  return run("qkv_norm_rope", a, as_stream(stream));
}

int mxk_qkv_norm_rope_scatter(const MxkHeadTensor* tensors_host, int n_tensors, int64_t S, int H, int D, float eps,
                              const float* cos, const float* sin, int groups, mxk_bf16* const* outs_host,
                              int64_t dst_row0, mxk_stream_t stream) {
  if (S <= 0 || n_tensors == 0) return MXK_OK;
  if (!tensors_host || !outs_host || n_tensors < 0 || n_tensors > kMaxTensors)
    return fail(MXK_ERR_INVALID_ARG, "qkv_norm_rope_scatter: n_tensors=%d (1..%d) or a null array", n_tensors, kMaxTensors);
  if (groups < 1 || groups > kMaxScatterGroups || H <= 0 || H % groups != 0)
    return fail(MXK_ERR_INVALID_ARG, "qkv_norm_rope_scatter: groups=%d (1..%d) must divide H=%d", groups, kMaxScatterGroups, H);
  if (dst_row0 < 0) return fail(MXK_ERR_INVALID_ARG, "qkv_norm_rope_scatter: dst_row0=%lld", (long long)dst_row0);
  RopeArgs a{};
  for (int i = 0; i < n_tensors; i++) {
    a.t[i] = tensors_host[i];
    for (int g = 0; g < groups; g++) {
      mxk_bf16* o = outs_host[i * groups + g];
      if (!o || !aligned(o, 16)) return fail(MXK_ERR_INVALID_ARG, "qkv_norm_rope_scatter: destination %d of tensor %d is null or not 16-byte aligned", g, i);
      a.scatter_out[i][g] = o;
    }
    a.t[i].out = a.scatter_out[i][0];
    if (int rc = check("qkv_norm_rope_scatter", a.t[i], H, D, cos, sin)) return rc;
  }
  a.n_tensors = n_tensors;
  a.S = S, a.H = H, a.D = D, a.eps = eps, a.cos = cos, a.sin = sin;
  a.scatter_groups = groups, a.heads_per_group = H / groups, a.scatter_row0 = dst_row0;
  if (!fast_ok(a))
    return fail(MXK_ERR_INVALID_ARG, "qkv_norm_rope_scatter: needs D in {32, 64, 128, 256}, 16-byte aligned inputs and tables, "
                "in_stride and col0 multiples of 8, rot a multiple of 8 (interleaved) or 16 (half)");
  return launch_register<true>("qkv_norm_rope_scatter", a, as_stream(stream));
}

}  // extern "C"
