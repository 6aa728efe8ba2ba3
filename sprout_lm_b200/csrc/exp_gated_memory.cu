// A matrix memory with exponential gates and a running maximum (the mLSTM recurrence), the two row kernels around the
// scan of csrc/gated_recurrence.cu.  All arithmetic is float32.
//
// Per head, with log gates i_t = cap * tanh(zi_t / cap) and f_t = logsigmoid(cap * tanh(zf_t / cap)) (zi, zf the gate
// projections plus their biases; cap <= 0: no cap) and a running maximum m (m before the first token is 0):
//     m_t = max(f_t + m_(t-1), i_t),   a_t = exp(f_t + m_(t-1) - m_t),   c_t = exp(i_t - m_t)
//     S_t = a_t S_(t-1) + c_t k_t v_t^T,   n_t = a_t n_(t-1) + c_t k_t
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// a_t and c_t never exceed 1.
//
//  * exp_gates:       m_t, a_t, c_t for every token of the step, from and into the requests' state slots (m per head).
//                     One block per (request, head): the gates of a tile of tokens side by side, the running maxima by one
//                     warp, 32 tokens at a time (m -> max(m + f, i) is a pair (f, i), and two steps in a row are the pair
//                     (f1 + f2, max(i1 + f2, i2)): a prefix scan over pairs with shuffles, then the carry from the tokens
//                     before), the exponentials side by side again.  Between two ways of cutting the tokens into steps the
//                     maxima differ by the rounding of the sums of f alone, and a shift of m moves S, n and exp(-m) alike.
//  * exp_memory_out:  the scan's rows [o | n . q | padding] per head into the mixer's gated, normed output:
//                     o / (max(|n . q|, exp(-m)) + 1e-6), divided by its root mean square over the head, times a weight,
//                     times sigmoid(gate), times out_scale.
#include "common.cuh"

namespace {

constexpr int GATE_TILE = 1024, GATE_THREADS = 128;

__device__ __forceinline__ float log_sigmoid_f(float z) { return -(fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z)))); }

__global__ void __launch_bounds__(GATE_THREADS)
exp_gates_kernel(const float* __restrict__ zi, const float* __restrict__ zf, int z_stride, const float* __restrict__ bias_i,
                 const float* __restrict__ bias_f, float cap, int heads, const int* __restrict__ q_start,
                 const int* __restrict__ state_slots, float* __restrict__ top_state, int num_slots, float* __restrict__ da,
                 float* __restrict__ dc, float* __restrict__ dm, int* status) {
  __shared__ float gi[GATE_TILE], gf[GATE_TILE], tops[GATE_TILE + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int begin = q_start[r], end = q_start[r + 1];
  if (begin >= end) return;
  const int slot = state_slots[r];
  if (slot < 0 || slot >= num_slots) {
    if (tid == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  float* mine = top_state + (size_t)slot * heads + h;
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  if (tid == 0) tops[0] = *mine;
  for (int t0 = begin; t0 < end; t0 += GATE_TILE) {
    const int n = min(GATE_TILE, end - t0);
    for (int j = tid; j < n; j += GATE_THREADS) {
      float a = zi[(size_t)(t0 + j) * z_stride + h] + bi, b = zf[(size_t)(t0 + j) * z_stride + h] + bf;
      if (cap > 0.f) {
        a = cap * tanhf(a * inv_cap);
        b = cap * tanhf(b * inv_cap);
      }
      gi[j] = a;
      gf[j] = log_sigmoid_f(b);
    }
    __syncthreads();
    if (tid < 32) {
      float carry = tops[0];
      for (int j0 = 0; j0 < n; j0 += 32) {
        const int j = j0 + tid;
        // beyond the tile's end: the pair that changes nothing, (0, -inf)
        float a = j < n ? gf[j] : 0.f, b = j < n ? gi[j] : -INFINITY;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const float ap = __shfl_up_sync(0xffffffffu, a, d), bp = __shfl_up_sync(0xffffffffu, b, d);
          if (tid >= d) {
            b = fmaxf(bp + a, b);
            a = ap + a;
          }
        }
        const float top = fmaxf(carry + a, b);
        if (j < n) tops[j + 1] = top;
        carry = __shfl_sync(0xffffffffu, top, 31);
      }
    }
    __syncthreads();
    for (int j = tid; j < n; j += GATE_THREADS) {
      const size_t at = (size_t)(t0 + j) * heads + h;
      const float before = tops[j], now = tops[j + 1];
      da[at] = expf(gf[j] + before - now);
      dc[at] = expf(gi[j] - now);
      dm[at] = now;
    }
    __syncthreads();
    if (tid == 0) tops[0] = tops[n];
  }
  if (tid == 0) *mine = tops[0];
}

// grid (tokens, heads).  o float32 [tokens, heads * o_cols]: per head vdim outputs, then n . q; gate float32 or T rows.
template <typename T, typename G>
__global__ void __launch_bounds__(128)
exp_memory_out_kernel(const float* __restrict__ o, int o_cols, const float* __restrict__ dm, const G* __restrict__ gate,
                      int gate_stride, const float* __restrict__ weight, T* __restrict__ out, int heads, int vdim, float eps,
                      float out_scale) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* src = o + ((size_t)t * heads + h) * o_cols;
  const float denominator = fmaxf(fabsf(src[vdim]), expf(-dm[(size_t)t * heads + h])) + 1e-6f;
  float squares = 0.f;
  for (int i = threadIdx.x; i < vdim; i += blockDim.x) {
    const float v = src[i] / denominator;
    squares = fmaf(v, v, squares);
  }
  const float r = out_scale / sqrtf(block_sum(squares, scratch) / (float)vdim + eps);
  const G* grow = gate + (size_t)t * gate_stride + (size_t)h * vdim;
  T* dst = out + ((size_t)t * heads + h) * vdim;
  for (int i = threadIdx.x; i < vdim; i += blockDim.x) {
    const float g = to_float(grow[i]);
    dst[i] = from_float<T>((src[i] / denominator) * r * weight[(size_t)h * vdim + i] * (1.0f / (1.0f + expf(-g))));
  }
}

}  // namespace

// zi, zf: float32 views [tokens, heads] with row stride z_stride; da, dc, dm: float32 [tokens, heads].
SPROUT_API int sprout_exp_gates(const float* zi, const float* zf, int z_stride, const float* bias_i, const float* bias_f, float cap,
                                int requests, int heads, const int* q_start, const int* state_slots, float* top_state,
                                int num_slots, float* da, float* dc, float* dm, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(zi && zf && q_start && state_slots && top_state && da && dc && dm && status, "exp_gates: null pointer");
  SPROUT_REQUIRE(requests > 0 && heads > 0 && heads <= 65535 && num_slots > 0 && z_stride >= heads, "exp_gates: bad sizes");
  sprout_launch(exp_gates_kernel, dim3(requests, heads), dim3(GATE_THREADS), 0, stream, zi, zf, z_stride, bias_i, bias_f, cap, heads,
                q_start, state_slots, top_state, num_slots, da, dc, dm, status);
  return sprout_check_launch("exp_gates");
}

SPROUT_API int sprout_exp_memory_out(const float* o, int o_cols, const float* dm, const void* gate, int gate_stride, int gate_f32,
                                     const float* weight, void* out, int dtype, int tokens, int heads, int vdim, float eps,
                                     float out_scale, cudaStream_t stream) {
  SPROUT_REQUIRE(o && dm && gate && weight && out, "exp_memory_out: null pointer");
  SPROUT_REQUIRE(tokens > 0 && heads > 0 && heads <= 65535 && vdim > 0 && o_cols > vdim && gate_stride >= heads * vdim && eps > 0.f,
                 "exp_memory_out: bad sizes");
  const dim3 grid(tokens, heads);
#define OUT(T, G)                                                                                                              \
  sprout_launch(exp_memory_out_kernel<T, G>, grid, dim3(128), 0, stream, o, o_cols, dm, (const G*)gate, gate_stride, weight, \
                (T*)out, heads, vdim, eps, out_scale)
  if (dtype == SPROUT_F32) {
    SPROUT_REQUIRE(gate_f32, "exp_memory_out: float32 outputs take float32 gates");
    OUT(float, float);
  } else if (dtype == SPROUT_BF16) {
    if (gate_f32) OUT(__nv_bfloat16, float); else OUT(__nv_bfloat16, __nv_bfloat16);
  } else {
    return sprout_fail("exp_memory_out: unknown dtype %d", dtype);
  }
#undef OUT
  return sprout_check_launch("exp_memory_out");
}
