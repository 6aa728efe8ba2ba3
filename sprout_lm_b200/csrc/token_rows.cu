// Row kernels of feed-forwards and of inputs that are added to the residual stream.  float32 arithmetic; the element
// type of activations (float or bfloat16) is a template parameter.
//
//  * unit_act:       out = act(gate) * up for rows laid out [gate: ff | up: ff], or out = act(in) for rows of ff elements;
//                    act = silu, the tanh form of gelu, or the exact (erf) gelu.
//  * side_gate:      out[t, j] = gelu_tanh(z[t, j]) * table[token[t], first + j]: a per-token row of a table gated by a
//                    projection of the stream.
//  * rms_add:        x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w: a normed row added to the stream.
//  * add_rows:       x[t] += vec (+ other[t]): a learned vector, and optionally another stream, added to every row.
//  * gated_rows_add: x[t] += sigmoid(logit[t]) * y[t]: a sublayer's float32 rows weighed by one number per token.
//  * narrow_rows:    the float32 stream in bfloat16, for a product that reads the stream itself.
#include "common.cuh"

namespace {

enum Activation : int { ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_GELU_ERF = 2 };

__device__ __forceinline__ float activate(float z, int act) {
  if (act == ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  if (act == ACT_GELU_ERF) return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
  return z / (1.0f + expf(-z));
}

template <typename T>
__global__ void __launch_bounds__(256)
unit_act_kernel(const T* __restrict__ in, int in_stride, T* __restrict__ out, int out_stride, long long count, int ff, int act,
                int gated) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / ff;
    const int j = (int)(e - r * ff);
    const T* row = in + (size_t)r * in_stride;
    float v = activate(to_float(row[j]), act);
    if (gated) v *= to_float(row[ff + j]);
    out[(size_t)r * out_stride + j] = from_float<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
side_gate_kernel(const T* __restrict__ z, int z_stride, const T* __restrict__ table, int table_stride, int first,
                 const int* __restrict__ tokens, int vocab, T* __restrict__ out, long long count, int dim, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / dim;
    const int j = (int)(e - t * dim);
    const int token = tokens[t];
    float v = 0.f;
    if (token < 0 || token >= vocab) atomicOr(status, SPROUT_STATUS_BAD_TOKEN);
    else v = activate(to_float(z[(size_t)t * z_stride + j]), ACT_GELU_TANH) * to_float(table[(size_t)token * table_stride + first + j]);
    out[e] = from_float<T>(v);
  }
}

// a block per row
__global__ void __launch_bounds__(256)
rms_add_kernel(const float* __restrict__ y, const float* __restrict__ weight, float* __restrict__ x, int width, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* src = y + (size_t)blockIdx.x * width;
  float squares = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) squares = fmaf(src[i], src[i], squares);
  const float r = 1.0f / sqrtf(block_sum(squares, scratch) / (float)width + eps);
  float* dst = x + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] += src[i] * r * weight[i];
}

__global__ void __launch_bounds__(256)
add_rows_kernel(float* __restrict__ x, const float* __restrict__ other, const float* __restrict__ vec, long long count, int width) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
    float v = x[e];
    if (other) v += other[e];
    x[e] = v + vec[e % width];
  }
}

__global__ void __launch_bounds__(256)
gated_rows_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ logits, int logit_stride,
                      long long count, int width) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / width;
    x[e] = fmaf(1.0f / (1.0f + expf(-logits[(size_t)t * logit_stride])), y[e], x[e]);
  }
}

__global__ void __launch_bounds__(256)
narrow_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long count) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x)
    out[e] = __float2bfloat16_rn(x[e]);
}

inline unsigned blocks_for(long long count) {
  const long long blocks = (count + 255) / 256;
  return (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
}

}  // namespace

SPROUT_API int sprout_unit_act(const void* in, int in_stride, void* out, int out_stride, int dtype, int rows, int ff, int act,
                               int gated, cudaStream_t stream) {
  SPROUT_REQUIRE(in && out && rows > 0 && ff > 0 && in_stride >= (gated ? 2 : 1) * ff && out_stride >= ff, "unit_act: bad arguments");
  SPROUT_REQUIRE(act >= ACT_SILU && act <= ACT_GELU_ERF, "unit_act: unknown activation %d", act);
  const long long count = (long long)rows * ff;
  if (dtype == SPROUT_F32)
    sprout_launch(unit_act_kernel<float>, dim3(blocks_for(count)), dim3(256), 0, stream, (const float*)in, in_stride, (float*)out,
                  out_stride, count, ff, act, gated);
  else if (dtype == SPROUT_BF16)
    sprout_launch(unit_act_kernel<__nv_bfloat16>, dim3(blocks_for(count)), dim3(256), 0, stream, (const __nv_bfloat16*)in, in_stride,
                  (__nv_bfloat16*)out, out_stride, count, ff, act, gated);
  else
    return sprout_fail("unit_act: unknown dtype %d", dtype);
  return sprout_check_launch("unit_act");
}

SPROUT_API int sprout_side_gate(const void* z, int z_stride, const void* table, int table_stride, int first, const int* tokens,
                                int vocab, void* out, int dtype, int rows, int dim, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(z && table && tokens && out && status && rows > 0 && dim > 0 && first >= 0 && first + dim <= table_stride &&
                 z_stride >= dim && vocab > 0, "side_gate: bad arguments");
  const long long count = (long long)rows * dim;
  if (dtype == SPROUT_F32)
    sprout_launch(side_gate_kernel<float>, dim3(blocks_for(count)), dim3(256), 0, stream, (const float*)z, z_stride,
                  (const float*)table, table_stride, first, tokens, vocab, (float*)out, count, dim, status);
  else if (dtype == SPROUT_BF16)
    sprout_launch(side_gate_kernel<__nv_bfloat16>, dim3(blocks_for(count)), dim3(256), 0, stream, (const __nv_bfloat16*)z, z_stride,
                  (const __nv_bfloat16*)table, table_stride, first, tokens, vocab, (__nv_bfloat16*)out, count, dim, status);
  else
    return sprout_fail("side_gate: unknown dtype %d", dtype);
  return sprout_check_launch("side_gate");
}

SPROUT_API int sprout_rms_add(const float* y, const float* weight, float* x, int rows, int width, float eps, cudaStream_t stream) {
  SPROUT_REQUIRE(y && weight && x && rows > 0 && width > 0 && eps > 0.f, "rms_add: bad arguments");
  sprout_launch(rms_add_kernel, dim3(rows), dim3(256), 0, stream, y, weight, x, width, eps);
  return sprout_check_launch("rms_add");
}

SPROUT_API int sprout_add_rows(float* x, const float* other, const float* vec, int rows, int width, cudaStream_t stream) {
  SPROUT_REQUIRE(x && vec && rows > 0 && width > 0, "add_rows: bad arguments");
  const long long count = (long long)rows * width;
  sprout_launch(add_rows_kernel, dim3(blocks_for(count)), dim3(256), 0, stream, x, other, vec, count, width);
  return sprout_check_launch("add_rows");
}

SPROUT_API int sprout_gated_rows_add(float* x, const float* y, const float* logits, int logit_stride, int rows, int width,
                                     cudaStream_t stream) {
  SPROUT_REQUIRE(x && y && logits && rows > 0 && width > 0 && logit_stride > 0, "gated_rows_add: bad arguments");
  const long long count = (long long)rows * width;
  sprout_launch(gated_rows_add_kernel, dim3(blocks_for(count)), dim3(256), 0, stream, x, y, logits, logit_stride, count, width);
  return sprout_check_launch("gated_rows_add");
}

SPROUT_API int sprout_narrow_rows(const float* x, void* out, long long count, cudaStream_t stream) {
  SPROUT_REQUIRE(x && out && count > 0, "narrow_rows: bad arguments");
  sprout_launch(narrow_rows_kernel, dim3(blocks_for(count)), dim3(256), 0, stream, x, (__nv_bfloat16*)out, count);
  return sprout_check_launch("narrow_rows");
}
