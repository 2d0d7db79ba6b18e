// The small helpers around the GEMMs: add_inplace_bf16, casts, axpy / axpby, bias adds and
// scatter_rows (reference: src/kernels/ops.cu:191-195, 235-242, 249-290).
#include "flat_map.cuh"

namespace mxk {
namespace {

struct AddBf16Op {  // x = bf16(x + y)
  static constexpr int VEC = 8;
  struct Frag { uint4 x, y; };
  bf16* x;
  const bf16* y;
  bool vector_ok() const { return aligned(x, 16) && aligned(y, 16); }
  __device__ Frag load(int64_t vi) const {
    return Frag{ld_stream(reinterpret_cast<const uint4*>(x) + vi), ld_stream(reinterpret_cast<const uint4*>(y) + vi)};
  }
  __device__ void finish(int64_t vi, const Frag& f) const {
    float a[8], b[8];
    unpack8(f.x, a);
    unpack8(f.y, b);
#pragma unroll
    for (int i = 0; i < 8; i++) a[i] += b[i];
    st_stream(reinterpret_cast<uint4*>(x) + vi, pack8(a));
  }
  __device__ void scalar(int64_t i) const { x[i] = __float2bfloat16(bf16_to_f(x[i]) + bf16_to_f(y[i])); }
};

struct F32ToBf16Op {
  static constexpr int VEC = 8;
  struct Frag { float4 a, b; };
  const float* x;
  bf16* y;
  bool vector_ok() const { return aligned(x, 16) && aligned(y, 16); }
  __device__ Frag load(int64_t vi) const {
    const float4* p = reinterpret_cast<const float4*>(x) + 2 * vi;
    return Frag{ld_stream(p), ld_stream(p + 1)};
  }
  __device__ void finish(int64_t vi, const Frag& f) const {
    const float v[8] = {f.a.x, f.a.y, f.a.z, f.a.w, f.b.x, f.b.y, f.b.z, f.b.w};
    st_stream(reinterpret_cast<uint4*>(y) + vi, pack8(v));
  }
  __device__ void scalar(int64_t i) const { y[i] = __float2bfloat16(x[i]); }
};

struct Bf16ToF32Op {
  static constexpr int VEC = 8;
  using Frag = uint4;
  const bf16* x;
  float* y;
  bool vector_ok() const { return aligned(x, 16) && aligned(y, 16); }
  __device__ Frag load(int64_t vi) const { return ld_stream(reinterpret_cast<const uint4*>(x) + vi); }
  __device__ void finish(int64_t vi, const Frag& f) const {
    float v[8];
    unpack8(f, v);
    float4* p = reinterpret_cast<float4*>(y) + 2 * vi;
    st_stream(p, make_float4(v[0], v[1], v[2], v[3]));
    st_stream(p + 1, make_float4(v[4], v[5], v[6], v[7]));
  }
  __device__ void scalar(int64_t i) const { y[i] = bf16_to_f(x[i]); }
};

struct AxpbyOp {  // x = a*x + b*y, or x += a*y when !scale_x
  static constexpr int VEC = 4;
  struct Frag { float4 x, y; };
  float* x;
  const float* y;
  float a, b;
  bool scale_x;
  bool vector_ok() const { return aligned(x, 16) && aligned(y, 16); }
  __device__ float f(float xv, float yv) const { return scale_x ? a * xv + b * yv : xv + a * yv; }
  __device__ Frag load(int64_t vi) const {
    return Frag{ld_stream(reinterpret_cast<const float4*>(x) + vi), ld_stream(reinterpret_cast<const float4*>(y) + vi)};
  }
  __device__ void finish(int64_t vi, const Frag& r) const {
    st_stream(reinterpret_cast<float4*>(x) + vi,
              make_float4(f(r.x.x, r.y.x), f(r.x.y, r.y.y), f(r.x.z, r.y.z), f(r.x.w, r.y.w)));
  }
  __device__ void scalar(int64_t i) const { x[i] = f(x[i], y[i]); }
};

// y[r, c] += bias[c]: each thread owns VEC consecutive columns (bias in registers) and walks a
// strip of rows; T is float or bf16.
template <class T>
__global__ void __launch_bounds__(256)
    add_bias_vec_kernel(T* __restrict__ y, const float* __restrict__ bias, int64_t rows, int dim,
                        int rows_per_chunk) {
  constexpr int VEC = sizeof(T) == 4 ? 4 : 8;
  constexpr int U = 4;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (col >= dim) return;
  float b[VEC];
#pragma unroll
  for (int q = 0; q < VEC / 4; q++) {
    float4 v = *reinterpret_cast<const float4*>(bias + col + 4 * q);
    b[4 * q] = v.x, b[4 * q + 1] = v.y, b[4 * q + 2] = v.z, b[4 * q + 3] = v.w;
  }
  const int64_t nchunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
  for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const int64_t r0 = c * rows_per_chunk;
    const int64_t r1 = r0 + rows_per_chunk < rows ? r0 + rows_per_chunk : rows;
    for (int64_t r = r0; r < r1; r += U) {
      uint4 raw[U];
#pragma unroll
      for (int k = 0; k < U; k++)
        if (r + k < r1) raw[k] = ld_stream(reinterpret_cast<const uint4*>(y + (r + k) * dim + col));
#pragma unroll
      for (int k = 0; k < U; k++) {
        if (r + k < r1) {
          uint4 o;
          if constexpr (sizeof(T) == 4) {
            o.x = __float_as_uint(__uint_as_float(raw[k].x) + b[0]);
            o.y = __float_as_uint(__uint_as_float(raw[k].y) + b[1]);
            o.z = __float_as_uint(__uint_as_float(raw[k].z) + b[2]);
            o.w = __float_as_uint(__uint_as_float(raw[k].w) + b[3]);
          } else {
            float v[8];
            unpack8(raw[k], v);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] += b[i];
            o = pack8(v);
          }
          st_stream(reinterpret_cast<uint4*>(y + (r + k) * dim + col), o);
        }
      }
    }
  }
}

template <class T>
__global__ void __launch_bounds__(256)
    add_bias_scalar_kernel(T* __restrict__ y, const float* __restrict__ bias, int64_t rows, int dim) {
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= dim) return;
  const float b = bias[i];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    if constexpr (sizeof(T) == 4) y[row * dim + i] += b;
    else y[row * dim + i] = __float2bfloat16(bf16_to_f(y[row * dim + i]) + b);
  }
}

template <class T>
int run_add_bias(const char* name, T* y, const float* bias, int64_t rows, int64_t dim, cudaStream_t s) {
  if (rows <= 0 || dim <= 0) return MXK_OK;
  if (!y || !bias) return fail(MXK_ERR_INVALID_ARG, "%s: null y or bias", name);
  if (dim > (int64_t(1) << 30)) return fail(MXK_ERR_INVALID_ARG, "%s: dim=%lld out of range", name, (long long)dim);
  constexpr int VEC = sizeof(T) == 4 ? 4 : 8;
  if (dim % VEC == 0 && aligned(y, 16) && aligned(bias, 16)) {
    const int rpc = 8;
    const unsigned gy = unsigned(ceil_div(dim / VEC, 256));
    const int64_t nchunks = ceil_div(rows, rpc);
    // one strip of rpc rows per CTA and as many CTAs as that takes: on B200 the streaming ops run faster handed out
    // tile by tile by the hardware than as one resident wave walking the rows (see run_flat)
    int64_t gx = nchunks < (int64_t(1) << 31) - 1 ? nchunks : (int64_t(1) << 31) - 1;
    if (gx < 1) gx = 1;
    add_bias_vec_kernel<T><<<dim3(unsigned(gx), gy), 256, 0, s>>>(y, bias, rows, int(dim), rpc);
  } else {
    const unsigned gy = unsigned(ceil_div(dim, 256));
    int64_t gx = rows < int64_t(sm_count()) * 16 ? rows : int64_t(sm_count()) * 16;
    add_bias_scalar_kernel<T><<<dim3(unsigned(gx), gy), 256, 0, s>>>(y, bias, rows, int(dim));
  }
  return after_launch(name);
}

// x[rows[i], :] = src[i, :] (or +=); one CTA row per source row, threads across the columns.
template <bool VEC4>
__global__ void __launch_bounds__(256)
    scatter_rows_kernel(float* __restrict__ x, int dim, const int32_t* __restrict__ rows,
                        const bf16* __restrict__ src, int64_t n, int add) {
  for (int64_t i = blockIdx.x; i < n; i += gridDim.x) {
    float* dst = x + int64_t(rows[i]) * dim;
    const bf16* sp = src + i * dim;
    if (VEC4) {
      for (int c = threadIdx.x * 4; c < dim; c += blockDim.x * 4) {
        float f[4];
        unpack4(*reinterpret_cast<const uint2*>(sp + c), f);
        float4* p = reinterpret_cast<float4*>(dst + c);
        float4 v = make_float4(f[0], f[1], f[2], f[3]);
        if (add) {
          float4 o = *p;
          v = make_float4(o.x + v.x, o.y + v.y, o.z + v.z, o.w + v.w);
        }
        *p = v;
      }
    } else {
      for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        const float v = bf16_to_f(sp[c]);
        dst[c] = add ? dst[c] + v : v;
      }
    }
  }
}

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int mxk_add_inplace_bf16(mxk_bf16* x, const mxk_bf16* y, int64_t n, mxk_stream_t stream) {
  if (n <= 0) return MXK_OK;
  if (!x || !y) return fail(MXK_ERR_INVALID_ARG, "add_inplace_bf16: null x or y");
  return run_flat("add_inplace_bf16", n, AddBf16Op{reinterpret_cast<bf16*>(x), reinterpret_cast<const bf16*>(y)},
                  as_stream(stream));
}

int mxk_f32_to_bf16(const float* x, mxk_bf16* y, int64_t n, mxk_stream_t stream) {
  if (n <= 0) return MXK_OK;
  if (!x || !y) return fail(MXK_ERR_INVALID_ARG, "f32_to_bf16: null x or y");
  return run_flat("f32_to_bf16", n, F32ToBf16Op{x, reinterpret_cast<bf16*>(y)}, as_stream(stream));
}

int mxk_bf16_to_f32(const mxk_bf16* x, float* y, int64_t n, mxk_stream_t stream) {
  if (n <= 0) return MXK_OK;
  if (!x || !y) return fail(MXK_ERR_INVALID_ARG, "bf16_to_f32: null x or y");
  return run_flat("bf16_to_f32", n, Bf16ToF32Op{reinterpret_cast<const bf16*>(x), y}, as_stream(stream));
}

int mxk_axpy_f32(float* x, const float* y, float a, int64_t n, mxk_stream_t stream) {
  if (n <= 0) return MXK_OK;
  if (!x || !y) return fail(MXK_ERR_INVALID_ARG, "axpy_f32: null x or y");
  return run_flat("axpy_f32", n, AxpbyOp{x, y, a, 0.f, false}, as_stream(stream));
}

int mxk_axpby_f32(float* x, const float* y, float a, float b, int64_t n, mxk_stream_t stream) {
  if (n <= 0) return MXK_OK;
  if (!x || !y) return fail(MXK_ERR_INVALID_ARG, "axpby_f32: null x or y");
  return run_flat("axpby_f32", n, AxpbyOp{x, y, a, b, true}, as_stream(stream));
}

int mxk_add_bias_bf16(mxk_bf16* y, const float* bias, int64_t rows, int64_t dim, mxk_stream_t stream) {
  return run_add_bias<bf16>("add_bias_bf16", reinterpret_cast<bf16*>(y), bias, rows, dim, as_stream(stream));
}

int mxk_add_bias_f32(float* y, const float* bias, int64_t rows, int64_t dim, mxk_stream_t stream) {
  return run_add_bias<float>("add_bias_f32", y, bias, rows, dim, as_stream(stream));
}

int mxk_scatter_rows(float* x, int64_t dim, const int32_t* rows, const mxk_bf16* src, int64_t n,
                     int add, mxk_stream_t stream) {
  if (n <= 0 || dim <= 0) return MXK_OK;
  if (!x || !rows || !src) return fail(MXK_ERR_INVALID_ARG, "scatter_rows: null x, rows or src");
  if (dim > (int64_t(1) << 30)) return fail(MXK_ERR_INVALID_ARG, "scatter_rows: dim=%lld out of range", (long long)dim);
  int64_t grid = n < int64_t(sm_count()) * 16 ? n : int64_t(sm_count()) * 16;
  const bf16* sp = reinterpret_cast<const bf16*>(src);
  if (dim % 4 == 0 && aligned(x, 16) && aligned(src, 8))
    scatter_rows_kernel<true><<<unsigned(grid), 256, 0, as_stream(stream)>>>(x, int(dim), rows, sp, n, add);
  else
    scatter_rows_kernel<false><<<unsigned(grid), 256, 0, as_stream(stream)>>>(x, int(dim), rows, sp, n, add);
  return after_launch("scatter_rows");
}

}  // extern "C"
