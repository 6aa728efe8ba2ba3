// Recurrent mixers whose decay comes from the input, and the row kernels around them.  All arithmetic is float32;
// the element type of the projections (float or bfloat16) is a template parameter.
//
//  * gated_scan:   per request and head, token by token:
//                      S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T,   o_t = S_t^T (q_scale q_t) + skip_h v_t
//                  with S [dim, vdim] float32 in the request's state slot.  Two ways to make a_t and c_t:
//                    per key channel (gated linear attention): a_t[i] = sigmoid(z_t[i] + bias[i])^(1/tau), c_t = 1;
//                    per head (a selective state space):      dt = softplus(z_t[h] + bias[h]), a_t[i] = exp(-exp(a_log[h]) dt),
//                                                             c_t = dt.
//                  q and k may be shared by the heads of a group (`groups` <= heads).  One block per (request, head,
//                  block of value columns); thread j owns column j of the state; the next token's q, k and decays are
//                  fetched while the current one is applied.  The order of operations per element is the tokens'
//                  order: the result does not depend on the cutting or on the batch.
//  * causal_conv:  y_t[c] = act(bias[c] + sum_j w[c][j] x_(t - (taps - 1 - j))[c]), zeros before the start of the
//                  sequence; the last taps - 1 inputs of a request live in its state slot [taps - 1, channels] and are
//                  read at the start of a portion and replaced at its end.
//  * gated_group_norm: rows in `groups` equal parts, each divided by its own root mean square, times a weight that
//                  repeats every `period` elements, times act(gate) before or after the norm.
//  * scaled_sum:   x += a y_1 + b y_2.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float silu_g(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_g(float z) { return 1.0f / (1.0f + expf(-z)); }

enum ScanDecay : int { DECAY_PER_CHANNEL = 0, DECAY_PER_HEAD = 1 };

template <typename T>
struct ScanParams {
  const T* q; int q_stride;            // [tokens, groups * dim]
  const T* k; int k_stride;            // [tokens, groups * dim]
  const T* v; int v_stride;            // [tokens, heads * vdim]
  const void* z; int z_stride, z_f32;  // per channel: [tokens, heads * dim]; per head: [tokens, heads]; of T, or float when z_f32
  const float* bias;                   // added to z: [heads * dim] or [heads]
  const float* a_log;                  // per head (per-head decay only)
  const float* skip;                   // per head, or null
  float inv_tau, q_scale;
  int mode, heads, groups, dim, vdim;
  const int* q_start; const int* state_slots; float* state; int num_slots;
  float* out;                          // [tokens, heads * vdim]
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(128)
gated_scan_kernel(const ScanParams<T> p) {
  extern __shared__ float smem[];
  const int cols = blockDim.x, dim = p.dim;
  float* S = smem;                                   // dim * cols
  float* token = S + (size_t)dim * cols;             // 2 buffers of [q | k | a], dim each
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int col = blockIdx.z * cols + threadIdx.x;
  const bool live = col < p.vdim;
  const int slot = p.state_slots[r];
  if (slot < 0 || slot >= p.num_slots) {
    if (threadIdx.x == 0) atomicOr(p.status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  const int g = h / (p.heads / p.groups);
  float* mine = p.state + (((size_t)slot * p.heads + h) * dim) * p.vdim;
  if (live)
    for (int i = 0; i < dim; i++) S[i * cols + threadIdx.x] = mine[(size_t)i * p.vdim + col];
  const float skip = p.skip ? p.skip[h] : 0.f;
  const float rate = p.mode == DECAY_PER_HEAD ? expf(p.a_log[h]) : 0.f;
  const int first = p.q_start[r], last = p.q_start[r + 1];

  auto z_at = [&](size_t index) { return p.z_f32 ? ((const float*)p.z)[index] : to_float(((const T*)p.z)[index]); };
  auto fetch = [&](int t, float* buf) {
    float step = 1.0f, decay = 1.0f;
    if (p.mode == DECAY_PER_HEAD) {
      step = softplus_f(z_at((size_t)t * p.z_stride + h) + p.bias[h]);
      decay = expf(-rate * step);
    }
    for (int i = threadIdx.x; i < dim; i += cols) {
      buf[i] = to_float(p.q[(size_t)t * p.q_stride + (size_t)g * dim + i]) * p.q_scale;
      buf[dim + i] = to_float(p.k[(size_t)t * p.k_stride + (size_t)g * dim + i]) * step;
      if (p.mode == DECAY_PER_CHANNEL) {
        const float zv = z_at((size_t)t * p.z_stride + (size_t)h * dim + i) + p.bias[(size_t)h * dim + i];
        decay = expf(-softplus_f(-zv) * p.inv_tau);              // sigmoid(z)^(1/tau) through its logarithm
      }
      buf[2 * dim + i] = decay;
    }
  };
  if (first < last) fetch(first, token);
  for (int t = first; t < last; t++) {
    float* cur = token + (size_t)((t - first) & 1) * 3 * dim;
    __syncthreads();                                 // this token's vectors are there; the other buffer is free
    if (t + 1 < last) fetch(t + 1, token + (size_t)((t + 1 - first) & 1) * 3 * dim);
    if (!live) continue;
    const float v = to_float(p.v[(size_t)t * p.v_stride + (size_t)h * p.vdim + col]);
    float o = skip * v;
    for (int i = 0; i < dim; i++) {
      const float s = fmaf(cur[2 * dim + i], S[i * cols + threadIdx.x], cur[dim + i] * v);
      S[i * cols + threadIdx.x] = s;
      o = fmaf(s, cur[i], o);
    }
    p.out[(size_t)t * p.heads * p.vdim + (size_t)h * p.vdim + col] = o;
  }
  if (live)
    for (int i = 0; i < dim; i++) mine[(size_t)i * p.vdim + col] = S[i * cols + threadIdx.x];
}

constexpr int CONV_MAX_TAPS = 8, CONV_TOKENS = 32;

// grid (request, blocks of 128 channels, blocks of CONV_TOKENS tokens); a thread walks its channel through its tokens
// with the last taps - 1 inputs in registers.  The block of a request's first tokens reads the state (before anything
// writes it) and is the one that writes the new state at its end.
template <typename T>
__global__ void __launch_bounds__(128)
causal_conv_kernel(const T* __restrict__ in, int in_stride, const float* __restrict__ weight, const float* __restrict__ bias,
                   T* __restrict__ out, int out_stride, const int* __restrict__ q_start, const int* __restrict__ state_slots,
                   float* __restrict__ state, int num_slots, int channels, int taps, int act, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  const int begin = q_start[r], end = q_start[r + 1];
  const int first = begin + blockIdx.z * CONV_TOKENS;
  if (first >= end || c >= channels) return;
  const int slot = state_slots[r];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  float* mine = state + (size_t)slot * (taps - 1) * channels + c;       // [taps - 1, channels], oldest first
  float w[CONV_MAX_TAPS], hist[CONV_MAX_TAPS];                           // hist[b]: the input b tokens back
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; j++) {
    w[j] = j < taps ? weight[(size_t)c * taps + j] : 0.f;
    hist[j] = 0.f;
  }
#pragma unroll
  for (int b = 1; b < CONV_MAX_TAPS; b++) {
    if (b >= taps) break;
    const int j = first - b;
    hist[b] = j >= begin ? to_float(in[(size_t)j * in_stride + c]) : mine[(size_t)(taps - 1 + (j - begin)) * channels];
  }
  float old[CONV_MAX_TAPS];                                              // the state as it was: old[b] is b tokens before the portion
#pragma unroll
  for (int b = 0; b < CONV_MAX_TAPS; b++) old[b] = hist[b];
  const float offset = bias ? bias[c] : 0.f;
  const int stop = min(first + CONV_TOKENS, end);
  for (int t = first; t < stop; t++) {
    hist[0] = to_float(in[(size_t)t * in_stride + c]);
    float y = offset;
#pragma unroll
    for (int b = CONV_MAX_TAPS - 1; b >= 0; b--)
      if (b < taps) y = fmaf(w[taps - 1 - b], hist[b], y);               // oldest input first
    out[(size_t)t * out_stride + c] = from_float<T>(act ? silu_g(y) : y);
#pragma unroll
    for (int b = CONV_MAX_TAPS - 1; b > 0; b--) hist[b] = hist[b - 1];
  }
  if (blockIdx.z != 0) return;
  // the new state: the last taps - 1 inputs of what the request has seen, oldest first
#pragma unroll
  for (int s = 0; s < CONV_MAX_TAPS - 1; s++) {
    if (s >= taps - 1) break;
    const int j = end - (taps - 1) + s;
    float value;
    if (j >= begin) {
      value = to_float(in[(size_t)j * in_stride + c]);
    } else {
      const int back = begin - j;                                        // 1 .. taps - 1 tokens before the portion
      value = 0.f;
#pragma unroll
      for (int b = 1; b < CONV_MAX_TAPS; b++)
        if (b == back) value = old[b];
    }
    mine[(size_t)s * channels] = value;
  }
}

// grid (rows, groups).  o float32 [rows, width]; gate rows of T with their own stride; out rows of T.
template <typename T>
__global__ void __launch_bounds__(128)
gated_group_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride, const float* __restrict__ weight,
                        int period, T* __restrict__ out, int width, int groups, float eps, int gate_first, int act) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int part = width / groups, base = blockIdx.y * part;
  const float* src = o + (size_t)blockIdx.x * width + base;
  const T* grow = gate + (size_t)blockIdx.x * gate_stride + base;
  float q = 0.f;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    float v = src[i];
    if (gate_first) {
      const float gv = to_float(grow[i]);
      v *= act ? silu_g(gv) : sigmoid_g(gv);
    }
    q = fmaf(v, v, q);
  }
  const float r = 1.0f / sqrtf(block_sum(q, scratch) / (float)part + eps);
  T* dst = out + (size_t)blockIdx.x * width + base;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float gv = to_float(grow[i]);
    const float factor = act ? silu_g(gv) : sigmoid_g(gv);
    const float v = gate_first ? (src[i] * factor) * r * weight[(base + i) % period] : src[i] * r * weight[(base + i) % period] * factor;
    dst[i] = from_float<T>(v);
  }
}

__global__ void scaled_sum_kernel(float* __restrict__ x, const float* __restrict__ y1, float a, const float* __restrict__ y2,
                                  float b, long long count) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
    x[i] += a * y1[i] + (y2 ? b * y2[i] : 0.f);
}

template <typename T>
int launch_scan(const ScanParams<T>& p, int requests, cudaStream_t stream) {
  int cols = p.vdim >= 128 ? 128 : (p.vdim + 31) / 32 * 32;
  // the state's columns of a block and two sets of token vectors must fit shared memory
  while (cols > 32 && ((size_t)p.dim * cols + 6 * p.dim) * sizeof(float) > 200 * 1024) cols -= 32;
  const size_t smem = ((size_t)p.dim * cols + 6 * p.dim) * sizeof(float);
  SPROUT_REQUIRE(smem <= 200 * 1024, "gated_scan: key vectors too long (%d)", p.dim);
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(gated_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return sprout_fail("gated_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
  }
  sprout_launch(gated_scan_kernel<T>, dim3(requests, p.heads, (p.vdim + cols - 1) / cols), dim3(cols), smem, stream, p);
  return sprout_check_launch("gated_scan");
}

}  // namespace

SPROUT_API int sprout_gated_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                                 const void* z, int z_stride, int z_f32, int dtype, const float* bias, const float* a_log, const float* skip,
                                 float inv_tau, float q_scale, int mode, int requests, int heads, int groups, int dim, int vdim,
                                 const int* q_start, const int* state_slots, float* state, int num_slots, float* out, int* status,
                                 cudaStream_t stream) {
  SPROUT_REQUIRE(q && k && v && z && bias && q_start && state_slots && state && out && status, "gated_scan: null pointer");
  SPROUT_REQUIRE(requests > 0 && heads > 0 && groups > 0 && heads % groups == 0 && dim > 0 && vdim > 0 && num_slots > 0,
                 "gated_scan: bad sizes");
  SPROUT_REQUIRE(mode == DECAY_PER_CHANNEL || (mode == DECAY_PER_HEAD && a_log), "gated_scan: unknown decay form");
  SPROUT_REQUIRE(heads <= 65535, "gated_scan: too many heads");
  if (dtype == SPROUT_F32) {
    ScanParams<float> p{(const float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, z, z_stride, z_f32,
                        bias, a_log, skip, inv_tau, q_scale, mode, heads, groups, dim, vdim, q_start, state_slots, state,
                        num_slots, out, status};
    return launch_scan(p, requests, stream);
  }
  if (dtype == SPROUT_BF16) {
    ScanParams<__nv_bfloat16> p{(const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v,
                                v_stride, z, z_stride, z_f32, bias, a_log, skip, inv_tau, q_scale, mode, heads,
                                groups, dim, vdim, q_start, state_slots, state, num_slots, out, status};
    return launch_scan(p, requests, stream);
  }
  return sprout_fail("gated_scan: unknown dtype %d", dtype);
}

// `max_q_len` bounds the tokens any request brings (it sizes the grid).
SPROUT_API int sprout_causal_conv(const void* in, int in_stride, const float* weight, const float* bias, void* out, int out_stride,
                                  int dtype, const int* q_start, const int* state_slots, float* state, int num_slots, int requests,
                                  int max_q_len, int channels, int taps, int act, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(in && weight && out && q_start && state_slots && state && status, "causal_conv: null pointer");
  SPROUT_REQUIRE(requests > 0 && max_q_len > 0 && channels > 0 && num_slots > 0, "causal_conv: bad sizes");
  SPROUT_REQUIRE(taps >= 2 && taps <= CONV_MAX_TAPS, "causal_conv: 2 to %d taps (got %d)", CONV_MAX_TAPS, taps);
  SPROUT_REQUIRE(in_stride >= channels && out_stride >= channels, "causal_conv: rows shorter than the channels");
  const dim3 grid(requests, (channels + 127) / 128, (max_q_len + CONV_TOKENS - 1) / CONV_TOKENS);
  SPROUT_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "causal_conv: too many channels or tokens");
  if (dtype == SPROUT_F32)
    sprout_launch(causal_conv_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, in_stride, weight, bias, (float*)out,
                  out_stride, q_start, state_slots, state, num_slots, channels, taps, act, status);
  else if (dtype == SPROUT_BF16)
    sprout_launch(causal_conv_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)in, in_stride, weight, bias,
                  (__nv_bfloat16*)out, out_stride, q_start, state_slots, state, num_slots, channels, taps, act, status);
  else
    return sprout_fail("causal_conv: unknown dtype %d", dtype);
  return sprout_check_launch("causal_conv");
}

SPROUT_API int sprout_gated_group_norm(const float* o, const void* gate, int gate_stride, const float* weight, int period, void* out,
                                       int dtype, int rows, int width, int groups, float eps, int gate_first, int act,
                                       cudaStream_t stream) {
  SPROUT_REQUIRE(o && gate && weight && out && rows > 0 && width > 0 && eps > 0, "gated_group_norm: bad arguments");
  SPROUT_REQUIRE(groups > 0 && groups <= 65535 && width % groups == 0 && period > 0 && gate_stride >= width,
                 "gated_group_norm: the row must divide into the groups, gate rows must hold the row");
  if (dtype == SPROUT_F32)
    sprout_launch(gated_group_norm_kernel<float>, dim3(rows, groups), dim3(128), 0, stream, o, (const float*)gate, gate_stride, weight,
                  period, (float*)out, width, groups, eps, gate_first, act);
  else if (dtype == SPROUT_BF16)
    sprout_launch(gated_group_norm_kernel<__nv_bfloat16>, dim3(rows, groups), dim3(128), 0, stream, o, (const __nv_bfloat16*)gate,
                  gate_stride, weight, period, (__nv_bfloat16*)out, width, groups, eps, gate_first, act);
  else
    return sprout_fail("gated_group_norm: unknown dtype %d", dtype);
  return sprout_check_launch("gated_group_norm");
}

SPROUT_API int sprout_scaled_sum(float* x, const float* y1, float a, const float* y2, float b, long long count, cudaStream_t stream) {
  SPROUT_REQUIRE(x && y1 && count > 0, "scaled_sum: bad arguments");
  const long long blocks = (count + 255) / 256;
  sprout_launch(scaled_sum_kernel, dim3((unsigned)(blocks < 148 * 8 ? blocks : 148 * 8)), dim3(256), 0, stream, x, y1, a, y2, b, count);
  return sprout_check_launch("scaled_sum");
}
