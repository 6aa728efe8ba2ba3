// Row kernels of layers that wrap every sublayer in two norms, all float32 arithmetic:
//  * layernorm:      out = (x - mean) / sqrt(var + eps) * w (+ b), var the mean of the squared deviations;
//                    rows may be selected by index.
//  * norm_add:       x += layernorm(y) * w_b, and, when asked, h = layernorm(x) * w_next of the new x:
//                    the norm after a sublayer, the residual sum and the norm before the next
//                    sublayer in one launch.
//  * gated_rmsnorm:  out = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate).
//  * relu2, glu_clamped: activations between the two products of a feed-forward.
// One block per row, or (rows of 128 to 4,096 elements in steps the kernels are built for) a warp per row with the row
// in registers; sums in a fixed order that depends on the row's width alone, so a row's result does not depend on
// what else is in the batch.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

// mean and 1 / sqrt(var + eps) of a row held in shared memory (two passes: the deviations are exact)
__device__ __forceinline__ void row_moments(const float* row, int width, float eps, float* scratch, float& mean, float& rstd) {
  float s = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) s += row[i];
  mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = row[i] - mean;
    q = fmaf(d, d, q);
  }
  rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)width + eps);
}

template <typename TO>
__global__ void __launch_bounds__(THREADS)
layernorm_kernel(const float* __restrict__ x, const float* __restrict__ gain, const float* __restrict__ bias,
                 TO* __restrict__ out, const int* __restrict__ rows, int width, float eps) {
  extern __shared__ float smem[];
  float* row = smem;                 // width
  float* scratch = smem + width;     // 33
  pdl_launch_dependents();
  pdl_wait();
  const size_t src = (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = x[src + i];
  __syncthreads();
  float mean, rstd;
  row_moments(row, width, eps, scratch, mean, rstd);
  TO* dst = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_float<TO>((row[i] - mean) * rstd * gain[i] + (bias ? bias[i] : 0.f));
}

template <typename TO>
__global__ void __launch_bounds__(THREADS)
norm_add_kernel(const float* __restrict__ y, const float* __restrict__ gain, float* __restrict__ x,
                const float* __restrict__ next_gain, TO* __restrict__ h, int width, float eps) {
  extern __shared__ float smem[];
  float* row = smem;
  float* scratch = smem + width;
  pdl_launch_dependents();
  pdl_wait();
  const size_t at = (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = y[at + i];
  __syncthreads();
  float mean, rstd;
  row_moments(row, width, eps, scratch, mean, rstd);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {      // each thread rewrites the elements it read
    const float v = x[at + i] + (row[i] - mean) * rstd * gain[i];
    x[at + i] = v;
    row[i] = v;
  }
  if (next_gain == nullptr) return;
  __syncthreads();
  row_moments(row, width, eps, scratch, mean, rstd);
  for (int i = threadIdx.x; i < width; i += blockDim.x) h[at + i] = from_float<TO>((row[i] - mean) * rstd * next_gain[i]);
}

// ---- rows of 128 * NV elements: a warp per row, the row in registers, 16-byte accesses, no block-wide barrier
template <typename TO>
__device__ __forceinline__ void store_four(TO* dst, float a, float b, float c, float d) {
  if (sizeof(TO) == 4) {
    *(float4*)dst = make_float4(a, b, c, d);
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2*)dst = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
  }
}

template <int NV>
__device__ __forceinline__ void warp_moments(const float4 (&v)[NV], float eps, float& mean, float& rstd) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; i++) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  mean = warp_sum(s) / (float)(NV * 128);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
    q += (a * a + b * b) + (c * c + d * d);
  }
  rstd = 1.0f / sqrtf(warp_sum(q) / (float)(NV * 128) + eps);
}

template <typename TO, int NV>
__global__ void __launch_bounds__(128)
layernorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ gain, const float* __restrict__ bias,
                      TO* __restrict__ out, const int* __restrict__ rows, int count, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= count) return;
  const float4* src = (const float4*)(x + (size_t)(rows ? rows[row] : row) * (NV * 128));
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) v[i] = src[i * 32 + lane];
  float mean, rstd;
  warp_moments<NV>(v, eps, mean, rstd);
  TO* dst = out + (size_t)row * (NV * 128);
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const float4 g = ((const float4*)gain)[i * 32 + lane];
    const float4 b = bias ? ((const float4*)bias)[i * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
    store_four<TO>(dst + (i * 32 + lane) * 4, (v[i].x - mean) * rstd * g.x + b.x, (v[i].y - mean) * rstd * g.y + b.y,
                   (v[i].z - mean) * rstd * g.z + b.z, (v[i].w - mean) * rstd * g.w + b.w);
  }
}

template <typename TO, int NV>
__global__ void __launch_bounds__(128)
norm_add_rows_kernel(const float* __restrict__ y, const float* __restrict__ gain, float* __restrict__ x,
                     const float* __restrict__ next_gain, TO* __restrict__ h, int count, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= count) return;
  const size_t at = (size_t)row * (NV * 128);
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) v[i] = ((const float4*)(y + at))[i * 32 + lane];
  float mean, rstd;
  warp_moments<NV>(v, eps, mean, rstd);
  float4* stream = (float4*)(x + at);
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const float4 g = ((const float4*)gain)[i * 32 + lane];
    float4 s = stream[i * 32 + lane];
    s.x += (v[i].x - mean) * rstd * g.x;
    s.y += (v[i].y - mean) * rstd * g.y;
    s.z += (v[i].z - mean) * rstd * g.z;
    s.w += (v[i].w - mean) * rstd * g.w;
    stream[i * 32 + lane] = s;
    v[i] = s;
  }
  if (next_gain == nullptr) return;
  warp_moments<NV>(v, eps, mean, rstd);
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const float4 g = ((const float4*)next_gain)[i * 32 + lane];
    store_four<TO>(h + at + (i * 32 + lane) * 4, (v[i].x - mean) * rstd * g.x, (v[i].y - mean) * rstd * g.y, (v[i].z - mean) * rstd * g.z,
                   (v[i].w - mean) * rstd * g.w);
  }
}

// 0: no such kernel for the width
inline int vectors_per_lane(int width) {
  if (width % 128) return 0;
  const int nv = width / 128;
  return (nv == 1 || nv == 2 || nv == 4 || nv == 6 || nv == 8 || nv == 12 || nv == 16 || nv == 24 || nv == 32) ? nv : 0;
}

#define SPROUT_FOR_NV(nv, CALL) \
  switch (nv) { case 1: CALL(1) break; case 2: CALL(2) break; case 4: CALL(4) break; case 6: CALL(6) break; case 8: CALL(8) break; \
                case 12: CALL(12) break; case 16: CALL(16) break; case 24: CALL(24) break; default: CALL(32) break; }

template <typename TG, typename TO>
__global__ void __launch_bounds__(THREADS)
gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gain, const TG* __restrict__ gate,
                     int gate_stride, TO* __restrict__ out, int width, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t at = (size_t)blockIdx.x * width;
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = o[at + i];
    q = fmaf(v, v, q);
  }
  const float r = 1.0f / sqrtf(block_sum(q, scratch) / (float)width + eps);
  const TG* grow = gate + (size_t)blockIdx.x * gate_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float g = to_float(grow[i]);
    out[at + i] = from_float<TO>(o[at + i] * r * gain[i] * (1.0f / (1.0f + expf(-g))));
  }
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ z, T* __restrict__ out, long long count) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_float(z[i]), 0.f);
    out[i] = from_float<T>(v * v);
  }
}

// rows of [gate (ff) | up (ff)] -> g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)
__device__ __forceinline__ float glu_value(float g, float u, float limit, float alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int ff, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const long long count = (long long)rows * ff;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / ff;
    const int j = (int)(i - r * ff);
    out[i] = from_float<T>(glu_value(to_float(gate_up[r * 2 * ff + j]), to_float(gate_up[r * 2 * ff + ff + j]), limit, alpha));
  }
}

// bfloat16 rows whose ff is a multiple of 8: eight elements a thread, 16-byte accesses
__global__ void glu_clamped_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int rows, int ff8,
                                       float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const long long count = (long long)rows * ff8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / ff8;
    const int j = (int)(i - r * ff8);
    const uint4 g = ((const uint4*)gate_up)[r * 2 * ff8 + j], u = ((const uint4*)gate_up)[r * 2 * ff8 + ff8 + j];
    const __nv_bfloat162* gp = (const __nv_bfloat162*)&g;
    const __nv_bfloat162* up = (const __nv_bfloat162*)&u;
    uint4 v;
    __nv_bfloat162* vp = (__nv_bfloat162*)&v;
#pragma unroll
    for (int e = 0; e < 4; e++)
      vp[e] = __floats2bfloat162_rn(glu_value(__low2float(gp[e]), __low2float(up[e]), limit, alpha),
                                    glu_value(__high2float(gp[e]), __high2float(up[e]), limit, alpha));
    ((uint4*)out)[i] = v;
  }
}

int grid_for(long long count) { return (int)((count + 255) / 256 < 148 * 8 ? (count + 255) / 256 : 148 * 8); }

}  // namespace

SPROUT_API int sprout_layernorm(const float* x, const float* gain, const float* bias, void* out, int out_dtype, const int* rows,
                                int count, int width, float eps, cudaStream_t stream) {
  SPROUT_REQUIRE(x && gain && out && count > 0 && width > 0 && eps > 0, "layernorm: bad arguments");
  SPROUT_REQUIRE(width <= 40000, "layernorm: rows of up to 40000 elements (got %d)", width);
  const int nv = vectors_per_lane(width);
  if (nv && (out_dtype == SPROUT_F32 || out_dtype == SPROUT_BF16) && (((uintptr_t)x | (uintptr_t)gain | (uintptr_t)bias | (uintptr_t)out) & 15) == 0) {
    const dim3 grid((count + 3) / 4);
#define CALL(N)                                                                                                                   \
    if (out_dtype == SPROUT_F32) sprout_launch(layernorm_rows_kernel<float, N>, grid, dim3(128), 0, stream, x, gain, bias, (float*)out, rows, count, eps); \
    else sprout_launch(layernorm_rows_kernel<__nv_bfloat16, N>, grid, dim3(128), 0, stream, x, gain, bias, (__nv_bfloat16*)out, rows, count, eps);
    SPROUT_FOR_NV(nv, CALL)
#undef CALL
    return sprout_check_launch("layernorm_rows");
  }
  const size_t smem = (size_t)(width + 34) * sizeof(float);
  if (out_dtype == SPROUT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sprout_launch(layernorm_kernel<float>, dim3(count), dim3(THREADS), smem, stream, x, gain, bias, (float*)out, rows, width, eps);
  } else if (out_dtype == SPROUT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sprout_launch(layernorm_kernel<__nv_bfloat16>, dim3(count), dim3(THREADS), smem, stream, x, gain, bias, (__nv_bfloat16*)out, rows, width, eps);
  } else {
    return sprout_fail("layernorm: unknown dtype %d", out_dtype);
  }
  return sprout_check_launch("layernorm");
}

// x [count, width] += layernorm(y) * gain; with next_gain also h = layernorm(x) * next_gain (h in h_dtype).
SPROUT_API int sprout_norm_add(const float* y, const float* gain, float* x, const float* next_gain, void* h, int h_dtype,
                               int count, int width, float eps, cudaStream_t stream) {
  SPROUT_REQUIRE(y && gain && x && count > 0 && width > 0 && eps > 0, "norm_add: bad arguments");
  SPROUT_REQUIRE((next_gain == nullptr) == (h == nullptr), "norm_add: the next norm's gain and its output go together");
  SPROUT_REQUIRE(width <= 40000, "norm_add: rows of up to 40000 elements (got %d)", width);
  const int nv = vectors_per_lane(width);
  if (nv && (h_dtype == SPROUT_F32 || h_dtype == SPROUT_BF16) &&
      (((uintptr_t)y | (uintptr_t)gain | (uintptr_t)x | (uintptr_t)next_gain | (uintptr_t)h) & 15) == 0) {
    const dim3 grid((count + 3) / 4);
#define CALL(N)                                                                                                                   \
    if (h_dtype == SPROUT_F32) sprout_launch(norm_add_rows_kernel<float, N>, grid, dim3(128), 0, stream, y, gain, x, next_gain, (float*)h, count, eps); \
    else sprout_launch(norm_add_rows_kernel<__nv_bfloat16, N>, grid, dim3(128), 0, stream, y, gain, x, next_gain, (__nv_bfloat16*)h, count, eps);
    SPROUT_FOR_NV(nv, CALL)
#undef CALL
    return sprout_check_launch("norm_add_rows");
  }
  const size_t smem = (size_t)(width + 34) * sizeof(float);
  if (h_dtype == SPROUT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sprout_launch(norm_add_kernel<float>, dim3(count), dim3(THREADS), smem, stream, y, gain, x, next_gain, (float*)h, width, eps);
  } else if (h_dtype == SPROUT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sprout_launch(norm_add_kernel<__nv_bfloat16>, dim3(count), dim3(THREADS), smem, stream, y, gain, x, next_gain, (__nv_bfloat16*)h, width, eps);
  } else {
    return sprout_fail("norm_add: unknown dtype %d", h_dtype);
  }
  return sprout_check_launch("norm_add");
}

// out [count, width] = o / rms(o) * gain * sigmoid(gate); gate rows have stride gate_stride and out's dtype.
SPROUT_API int sprout_gated_rmsnorm(const float* o, const float* gain, const void* gate, int gate_stride, void* out, int dtype,
                                    int count, int width, float eps, cudaStream_t stream) {
  SPROUT_REQUIRE(o && gain && gate && out && count > 0 && width > 0 && eps > 0 && gate_stride >= width, "gated_rmsnorm: bad arguments");
  if (dtype == SPROUT_F32)
    sprout_launch(gated_rmsnorm_kernel<float, float>, dim3(count), dim3(THREADS), 0, stream, o, gain, (const float*)gate,
                  gate_stride, (float*)out, width, eps);
  else if (dtype == SPROUT_BF16)
    sprout_launch(gated_rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(count), dim3(THREADS), 0, stream, o, gain,
                  (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, width, eps);
  else
    return sprout_fail("gated_rmsnorm: unknown dtype %d", dtype);
  return sprout_check_launch("gated_rmsnorm");
}

SPROUT_API int sprout_relu2(const void* z, void* out, int dtype, long long count, cudaStream_t stream) {
  SPROUT_REQUIRE(z && out && count > 0, "relu2: bad arguments");
  if (dtype == SPROUT_F32)
    sprout_launch(relu2_kernel<float>, dim3(grid_for(count)), dim3(256), 0, stream, (const float*)z, (float*)out, count);
  else if (dtype == SPROUT_BF16)
    sprout_launch(relu2_kernel<__nv_bfloat16>, dim3(grid_for(count)), dim3(256), 0, stream, (const __nv_bfloat16*)z,
                  (__nv_bfloat16*)out, count);
  else
    return sprout_fail("relu2: unknown dtype %d", dtype);
  return sprout_check_launch("relu2");
}

SPROUT_API int sprout_glu_clamped(const void* gate_up, void* out, int dtype, int rows, int ff, float limit, float alpha,
                                  cudaStream_t stream) {
  SPROUT_REQUIRE(gate_up && out && rows > 0 && ff > 0 && limit > 0, "glu_clamped: bad arguments");
  const long long count = (long long)rows * ff;
  if (dtype == SPROUT_F32)
    sprout_launch(glu_clamped_kernel<float>, dim3(grid_for(count)), dim3(256), 0, stream, (const float*)gate_up, (float*)out,
                  rows, ff, limit, alpha);
  else if (dtype == SPROUT_BF16 && ff % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0)
    sprout_launch(glu_clamped_vec_kernel, dim3(grid_for(count / 8)), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up,
                  (__nv_bfloat16*)out, rows, ff / 8, limit, alpha);
  else if (dtype == SPROUT_BF16)
    sprout_launch(glu_clamped_kernel<__nv_bfloat16>, dim3(grid_for(count)), dim3(256), 0, stream,
                  (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, rows, ff, limit, alpha);
  else
    return sprout_fail("glu_clamped: unknown dtype %d", dtype);
  return sprout_check_launch("glu_clamped");
}
