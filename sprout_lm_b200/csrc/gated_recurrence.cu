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
//                  block of value columns) with its part of the state in registers; the tokens' vectors come through
//                  shared memory a few tokens at a time.  The order of operations per element is the tokens' order:
//                  the result does not depend on the cutting or on the batch.
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

constexpr int SCAN_THREADS = 128, SCAN_MAX_TOKENS = 8;

// A block of SCAN_THREADS threads owns (request, head, `cb` value columns).  The state's rows are dealt to `slices`
// lanes of a warp (a power of two): the thread of slice s and column c keeps rows s, s + slices, s + 2 slices, ... of
// column c in ROWS registers, so the whole state of the block stays in registers from the first token to the last.
// Tokens come `batch` at a time (batch * slices <= 64): while the threads walk a batch's tokens over their registers,
// the next batch's q, k, decay inputs and values are on their way from memory into registers; at the batch's end
// they are turned into float32 vectors in shared memory ([q_scale q | c k | a] per row).  The slices of a column add
// their parts of o with shuffles.  Each element of S sees S <- fma(a, S, (c k) v) once per token in the tokens'
// order, so the result does not depend on the cutting or on the batch.
template <typename T, int ROWS>
__global__ void __launch_bounds__(SCAN_THREADS)
gated_scan_kernel(const ScanParams<T> p, int slices_log2, int batch) {
  constexpr int EPT = ROWS / 2;                      // row vectors a thread fetches per batch: batch * slices * ROWS / threads
  constexpr int VPT = SCAN_MAX_TOKENS;               // values a thread fetches per batch: batch * cb / threads <= batch
  extern __shared__ float4 scan_smem[];
  const int slices = 1 << slices_log2, dim = p.dim;
  const int rows_log2 = slices_log2 + (ROWS == 16 ? 4 : 5), rows_pad = 1 << rows_log2;
  const int cb_log2 = 7 - slices_log2, cb = 1 << cb_log2;
  float4* tok = scan_smem;                                             // [batch][rows_pad]: (q, k, a, -)
  float* vt = reinterpret_cast<float*>(tok + (size_t)batch * rows_pad);  // [batch][cb]
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int slice = tid & (slices - 1), col_local = tid >> slices_log2;
  const int col = blockIdx.z * cb + col_local;
  const bool live = col < p.vdim;
  const int slot = p.state_slots[r];
  if (slot < 0 || slot >= p.num_slots) {
    if (tid == 0) atomicOr(p.status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  const int g = h / (p.heads / p.groups);
  const bool per_head = p.mode == DECAY_PER_HEAD;
  float* mine = p.state + (((size_t)slot * p.heads + h) * dim) * p.vdim;
  float S[ROWS];
#pragma unroll
  for (int j = 0; j < ROWS; j++) {
    const int row = j * slices + slice;
    S[j] = (live && row < dim) ? mine[(size_t)row * p.vdim + col] : 0.f;
  }
  const float skip = p.skip ? p.skip[h] : 0.f;
  const float rate = per_head ? expf(p.a_log[h]) : 0.f;
  const int first = p.q_start[r], last = p.q_start[r + 1];
  auto z_at = [&](size_t index) { return p.z_f32 ? ((const float*)p.z)[index] : to_float(((const T*)p.z)[index]); };

  float rq[EPT], rk[EPT], rz[EPT], rv[VPT];
  auto fetch = [&](int t0) {                          // loads only: nothing waits for them here
    const int n = min(batch, last - t0);
#pragma unroll
    for (int u = 0; u < EPT; u++) {
      const int e = tid + u * SCAN_THREADS, tt = e >> rows_log2, i = e & (rows_pad - 1);
      rq[u] = rk[u] = rz[u] = 0.f;
      if (tt < n && i < dim) {
        const size_t t = (size_t)(t0 + tt);
        rq[u] = to_float(p.q[t * p.q_stride + (size_t)g * dim + i]);
        rk[u] = to_float(p.k[t * p.k_stride + (size_t)g * dim + i]);
        rz[u] = per_head ? z_at(t * p.z_stride + h) : z_at(t * p.z_stride + (size_t)h * dim + i);
      }
    }
#pragma unroll
    for (int u = 0; u < VPT; u++) {
      const int e = tid + u * SCAN_THREADS, tt = e >> cb_log2, column = blockIdx.z * cb + (e & (cb - 1));
      rv[u] = (tt < n && column < p.vdim) ? to_float(p.v[(size_t)(t0 + tt) * p.v_stride + (size_t)h * p.vdim + column]) : 0.f;
    }
  };
  if (first < last) fetch(first);
  for (int t0 = first; t0 < last; t0 += batch) {
    const int n = min(batch, last - t0);
    __syncthreads();                                   // the batch before has been read by everyone
#pragma unroll
    for (int u = 0; u < EPT; u++) {
      const int e = tid + u * SCAN_THREADS, tt = e >> rows_log2, i = e & (rows_pad - 1);
      if (tt >= n) break;
      float4 x = make_float4(0.f, 0.f, 1.f, 0.f);      // rows beyond dim stay zero
      if (i < dim) {
        float step = 1.0f, decay;
        if (per_head) {
          step = softplus_f(rz[u] + p.bias[h]);
          decay = expf(-rate * step);
        } else {
          decay = expf(-softplus_f(-(rz[u] + p.bias[(size_t)h * dim + i])) * p.inv_tau);  // sigmoid(z)^(1/tau) through its logarithm
        }
        x.x = rq[u] * p.q_scale;
        x.y = rk[u] * step;
        x.z = decay;
      }
      tok[e] = x;
    }
#pragma unroll
    for (int u = 0; u < VPT; u++) {
      const int e = tid + u * SCAN_THREADS;
      if (e < (n << cb_log2)) vt[e] = rv[u];
    }
    __syncthreads();
    if (t0 + batch < last) fetch(t0 + batch);          // in flight while this batch is applied
    for (int tt = 0; tt < n; tt++) {
      const float v = vt[(tt << cb_log2) + col_local];
      const float4* cur = tok + ((size_t)tt << rows_log2) + slice;
      float o = 0.f;
#pragma unroll
      for (int j = 0; j < ROWS; j++) {
        const float4 x = cur[j << slices_log2];
        const float s = fmaf(x.z, S[j], x.y * v);
        S[j] = s;
        o = fmaf(s, x.x, o);
      }
      for (int d = slices >> 1; d > 0; d >>= 1) o += __shfl_xor_sync(0xffffffffu, o, d);
      if (slice == 0 && live) p.out[(size_t)(t0 + tt) * p.heads * p.vdim + (size_t)h * p.vdim + col] = fmaf(skip, v, o);
    }
  }
#pragma unroll
  for (int j = 0; j < ROWS; j++) {
    const int row = j * slices + slice;
    if (live && row < dim) mine[(size_t)row * p.vdim + col] = S[j];
  }
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
  // rows per thread: 16 up to 512 key channels, 32 up to 1024; the slices of a column are lanes of one warp
  const int rows = p.dim <= 16 * 32 ? 16 : 32;
  SPROUT_REQUIRE(p.dim <= rows * 32, "gated_scan: key vectors too long (%d)", p.dim);
  int slices_log2 = 0;
  while ((rows << slices_log2) < p.dim) slices_log2++;
  const int slices = 1 << slices_log2, cb = SCAN_THREADS / slices;
  const int batch = 64 / slices < SCAN_MAX_TOKENS ? 64 / slices : SCAN_MAX_TOKENS;
  const size_t smem = (size_t)batch * ((size_t)rows * slices * sizeof(float4) + (size_t)cb * sizeof(float));
  const dim3 grid(requests, p.heads, (p.vdim + cb - 1) / cb);
  SPROUT_REQUIRE(grid.z <= 65535, "gated_scan: too many value columns");
  if (rows == 16)
    sprout_launch(gated_scan_kernel<T, 16>, grid, dim3(SCAN_THREADS), smem, stream, p, slices_log2, batch);
  else
    sprout_launch(gated_scan_kernel<T, 32>, grid, dim3(SCAN_THREADS), smem, stream, p, slices_log2, batch);
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
