// Row kernels of feed-forwards and of inputs that are added to the residual stream.  float32 arithmetic; the element
// type of activations (float or bfloat16) is a template parameter.
//
//  * unit_act:       out = act(gate) * up for rows laid out [gate: ff | up: ff], or out = act(in) for rows of ff elements;
//                    act = silu, the tanh form of gelu, or the exact (erf) gelu.  Optionally every row is also multiplied
//                    by sigmoid(logit[row]): a gate per token on a sublayer whose last step is linear.
//  * side_input_few: the whole per-layer token input for a handful of tokens in two launches (see side_gate, rms_add).
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
                int gated, const float* __restrict__ row_logits, int logit_stride) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / ff;
    const int j = (int)(e - r * ff);
    const T* row = in + (size_t)r * in_stride;
    float v = activate(to_float(row[j]), act);
    if (gated) v *= to_float(row[ff + j]);
    if (row_logits) v *= 1.0f / (1.0f + expf(-row_logits[(size_t)r * logit_stride]));
    out[(size_t)r * out_stride + j] = from_float<T>(v);
  }
}

// bfloat16 rows of 16-byte multiples: eight elements a thread, the same arithmetic
__global__ void __launch_bounds__(256)
unit_act_vec_kernel(const __nv_bfloat16* __restrict__ in, int in_stride, __nv_bfloat16* __restrict__ out, int out_stride, long long groups,
                    int ff, int act, int gated, const float* __restrict__ row_logits, int logit_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = ff / 8;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < groups; e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / per_row;
    const int j = (int)(e - r * per_row) * 8;
    const __nv_bfloat16* row = in + (size_t)r * in_stride;
    const uint4 a = *reinterpret_cast<const uint4*>(row + j);
    uint4 b = make_uint4(0, 0, 0, 0);
    if (gated) b = *reinterpret_cast<const uint4*>(row + ff + j);
    const float scale = row_logits ? 1.0f / (1.0f + expf(-row_logits[(size_t)r * logit_stride])) : 1.0f;
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 result;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 x = __bfloat1622float2(ap[i]), u = __bfloat1622float2(bp[i]);
      float v0 = activate(x.x, act), v1 = activate(x.y, act);
      if (gated) { v0 *= u.x; v1 *= u.y; }
      rp[i] = __floats2bfloat162_rn(v0 * scale, v1 * scale);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * out_stride + j) = result;
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

// The per-layer token input for a handful of tokens, in two launches that keep many SMs busy.
//  side_few_gate: grid (tokens, blocks of SIDE_GATE_OUTPUTS outputs), a warp per output: z = W_gate x over the stream's row as T
//                 holds it (float32 sums, the lanes added in a fixed order), g = gelu_tanh(z) * the token's table row (float32 out).
//  side_few_proj: a block per token, a thread per output column: y = W_proj g with the row of W_proj in the thread's own
//                 loads, then x += y / rms(y) * w.
// Intermediate results are rounded to T where the separate products would round them.
constexpr int SIDE_MAX_DIM = 512, SIDE_GATE_OUTPUTS = 8, SIDE_PROJ_THREADS = 512;

template <typename T>
__global__ void __launch_bounds__(SIDE_GATE_OUTPUTS * 32)
side_few_gate_kernel(const float* __restrict__ x, const T* __restrict__ w_gate, const T* __restrict__ table, int table_stride, int first,
                     const int* __restrict__ tokens, int vocab, float* __restrict__ g, int width, int dim, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, j = blockIdx.y * SIDE_GATE_OUTPUTS + (threadIdx.x >> 5);
  if (j >= dim) return;
  const int token = tokens[t];
  if (token < 0 || token >= vocab) {
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, SPROUT_STATUS_BAD_TOKEN);
    if (lane == 0) g[(size_t)t * dim + j] = 0.f;
    return;
  }
  const float* row = x + (size_t)t * width;
  const T* w = w_gate + (size_t)j * width;
  float sum = 0.f;
  if ((width & 3) == 0 && sizeof(T) == 2) {
    for (int k = lane * 4; k < width; k += 128) {
      const float4 xv = *reinterpret_cast<const float4*>(row + k);
      const uint2 wv = *reinterpret_cast<const uint2*>(w + k);
      const float2 w01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv.x));
      const float2 w23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv.y));
      sum = fmaf(to_float(from_float<T>(xv.x)), w01.x, sum);
      sum = fmaf(to_float(from_float<T>(xv.y)), w01.y, sum);
      sum = fmaf(to_float(from_float<T>(xv.z)), w23.x, sum);
      sum = fmaf(to_float(from_float<T>(xv.w)), w23.y, sum);
    }
  } else {
    for (int k = lane; k < width; k += 32) sum = fmaf(to_float(from_float<T>(row[k])), to_float(w[k]), sum);
  }
  sum = warp_sum(sum);
  if (lane == 0) {
    const float z = to_float(from_float<T>(sum));
    g[(size_t)t * dim + j] = to_float(from_float<T>(activate(z, ACT_GELU_TANH) * to_float(table[(size_t)token * table_stride + first + j])));
  }
}

template <typename T>
__global__ void __launch_bounds__(SIDE_PROJ_THREADS)
side_few_proj_kernel(float* __restrict__ x, const float* __restrict__ g, const T* __restrict__ w_proj, const float* __restrict__ weight,
                     int width, int dim, float eps) {
  extern __shared__ float side_smem[];
  float* ys = side_smem;                 // width
  __shared__ float gs[SIDE_MAX_DIM];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int k = threadIdx.x; k < dim; k += SIDE_PROJ_THREADS) gs[k] = g[(size_t)t * dim + k];
  __syncthreads();
  float squares = 0.f;
  for (int n = threadIdx.x; n < width; n += SIDE_PROJ_THREADS) {
    const T* w = w_proj + (size_t)n * dim;
    float sum = 0.f;
    if ((dim & 7) == 0 && sizeof(T) == 2) {
      for (int k = 0; k < dim; k += 8) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const float2 f = __bfloat1622float2(wp[i]);
          sum = fmaf(gs[k + 2 * i], f.x, sum);
          sum = fmaf(gs[k + 2 * i + 1], f.y, sum);
        }
      }
    } else {
      for (int k = 0; k < dim; k++) sum = fmaf(gs[k], to_float(w[k]), sum);
    }
    ys[n] = sum;
    squares = fmaf(sum, sum, squares);
  }
  const float r = 1.0f / sqrtf(block_sum(squares, scratch) / (float)width + eps);
  float* row = x + (size_t)t * width;
  for (int n = threadIdx.x; n < width; n += SIDE_PROJ_THREADS) row[n] += ys[n] * r * weight[n];
}

inline unsigned blocks_for(long long count) {
  const long long blocks = (count + 255) / 256;
  return (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
}

}  // namespace

// g: float32 scratch [rows, dim].
SPROUT_API int sprout_side_input_few(float* x, const void* w_gate, const void* w_proj, const float* weight, const void* table,
                                     int table_stride, int first, const int* tokens, int vocab, int dtype, int rows, int width,
                                     int dim, float eps, float* g, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(x && w_gate && w_proj && weight && table && tokens && g && status, "side_input_few: null pointer");
  SPROUT_REQUIRE(rows > 0 && width > 0 && dim > 0 && dim <= SIDE_MAX_DIM && first >= 0 && first + dim <= table_stride && vocab > 0 &&
                 eps > 0.f, "side_input_few: bad sizes (dim up to %d)", SIDE_MAX_DIM);
  const size_t smem = (size_t)width * sizeof(float);
  SPROUT_REQUIRE(smem <= 40 * 1024, "side_input_few: rows of up to 10240 elements");
  SPROUT_REQUIRE(dtype != SPROUT_BF16 || (((uintptr_t)w_gate | (uintptr_t)w_proj | (uintptr_t)x) & 15) == 0,
                 "side_input_few: buffers must start on 16-byte boundaries");
  const dim3 gate_grid(rows, (dim + SIDE_GATE_OUTPUTS - 1) / SIDE_GATE_OUTPUTS);
  SPROUT_REQUIRE(gate_grid.y <= 65535, "side_input_few: too many outputs");
  if (dtype == SPROUT_F32) {
    sprout_launch(side_few_gate_kernel<float>, gate_grid, dim3(SIDE_GATE_OUTPUTS * 32), 0, stream, (const float*)x, (const float*)w_gate,
                  (const float*)table, table_stride, first, tokens, vocab, g, width, dim, status);
    if (int rc = sprout_check_launch("side_input_few (gate)")) return rc;
    sprout_launch(side_few_proj_kernel<float>, dim3(rows), dim3(SIDE_PROJ_THREADS), smem, stream, x, (const float*)g, (const float*)w_proj,
                  weight, width, dim, eps);
  } else if (dtype == SPROUT_BF16) {
    sprout_launch(side_few_gate_kernel<__nv_bfloat16>, gate_grid, dim3(SIDE_GATE_OUTPUTS * 32), 0, stream, (const float*)x,
                  (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)table, table_stride, first, tokens, vocab, g, width, dim, status);
    if (int rc = sprout_check_launch("side_input_few (gate)")) return rc;
    sprout_launch(side_few_proj_kernel<__nv_bfloat16>, dim3(rows), dim3(SIDE_PROJ_THREADS), smem, stream, x, (const float*)g,
                  (const __nv_bfloat16*)w_proj, weight, width, dim, eps);
  } else {
    return sprout_fail("side_input_few: unknown dtype %d", dtype);
  }
  return sprout_check_launch("side_input_few (projection)");
}

SPROUT_API int sprout_unit_act(const void* in, int in_stride, void* out, int out_stride, int dtype, int rows, int ff, int act,
                               int gated, const float* row_logits, int logit_stride, cudaStream_t stream) {
  SPROUT_REQUIRE(in && out && rows > 0 && ff > 0 && in_stride >= (gated ? 2 : 1) * ff && out_stride >= ff, "unit_act: bad arguments");
  SPROUT_REQUIRE(act >= ACT_SILU && act <= ACT_GELU_ERF, "unit_act: unknown activation %d", act);
  const long long count = (long long)rows * ff;
  if (dtype == SPROUT_F32)
    sprout_launch(unit_act_kernel<float>, dim3(blocks_for(count)), dim3(256), 0, stream, (const float*)in, in_stride, (float*)out,
                  out_stride, count, ff, act, gated, row_logits, logit_stride);
  else if (dtype == SPROUT_BF16 && ff % 8 == 0 && in_stride % 8 == 0 && out_stride % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0)
    sprout_launch(unit_act_vec_kernel, dim3(blocks_for(count / 8)), dim3(256), 0, stream, (const __nv_bfloat16*)in, in_stride,
                  (__nv_bfloat16*)out, out_stride, count / 8, ff, act, gated, row_logits, logit_stride);
  else if (dtype == SPROUT_BF16)
    sprout_launch(unit_act_kernel<__nv_bfloat16>, dim3(blocks_for(count)), dim3(256), 0, stream, (const __nv_bfloat16*)in, in_stride,
                  (__nv_bfloat16*)out, out_stride, count, ff, act, gated, row_logits, logit_stride);
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
