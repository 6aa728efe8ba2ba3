// A routed feed-forward (mixture of experts), all on the device: no count ever travels to the host.
//
//  * moe_route:    per token z = W_router h (float32), s = softmax(z) over all router outputs,
//                  choice = s + correction; the `top` largest choices (lowest index first among equals) are
//                  taken; weight = s / (sum of the taken s + 1e-20) * scale.  Router outputs from
//                  `experts` on are identity experts (their output is the token's h).  Counts the rows
//                  of each real expert.  Options: the outputs form `group_count` equal groups of neighbours, a group's
//                  score is its largest s, and only outputs of the `group_keep` best groups can be taken; weights that
//                  are the scores themselves (not renormalised); `extra` further rows of the router matrix whose
//                  products are handed out as they are (a gate beside the router, in the same 32-bit product).
//  * moe_arrange:  offsets of the experts' row ranges, every taken (token, place) of a real expert put
//                  into its expert's range (`sorted`), and where it went (`place_of`).
//  * moe_up / moe_down (plain): the experts' two products on CUDA cores over the arranged rows, every
//                  output element summed in ascending k by one warp: act = f(W_gate a, W_up a),
//                  rows = W_down act, f(g, u) = g' sigmoid(alpha g') (u' + 1), g' = min(g, limit),
//                  u' = clamp(u, -limit, limit); or, for experts without a gate, act = gelu(W_up a) (the exact, erf form)
//                  with a matrix of ff rows per expert.
//  * moe_up / moe_down (mma):   the same two products on tensor cores (bfloat16, `mma.sync.m16n8k16`, float32
//                  accumulation): a CTA makes 128 arranged rows of one expert x 128 columns, K in steps of 64
//                  through a three-stage cp.async ring; the tile list follows the experts' row counts on the
//                  device.  In the up product a tile holds 64 gate columns and the 64 up columns that go with
//                  them, so the activation is applied to the accumulators.
//  * moe_few:      the same two products for steps of at most 8 tokens (bfloat16): a CTA per (expert, 32 output columns)
//                  keeps the expert's few rows in shared memory and streams every weight row once for all of them.
//  * moe_combine:  y[t] += sum over the token's places of weight * (identity ? h[t] : its row).
#include "attention_bf16.cuh"

using namespace sprout_attn;

namespace {

// threads of a router block: 32 warps, so that the router's rows are walked by as many warps as the SM holds (a block's time is
// the latency of its rounds over the outputs: 33 outputs are 2 rounds of 32 warps, 5 of 8)
constexpr int ROUTE_THREADS = 1024;

// A block takes ROUTE_TOKENS tokens (8 in steps of many tokens, 1 in steps of few, where blocks are scarce; a token's
// sums are the same in both): the 32 warps share the router's outputs (warp w takes outputs w, w + 32, ...) and apply every
// weight they load to all 8 tokens; a lane sums its own elements in ascending order (four neighbours of every 128 where the rows
// are multiples of four, else every 32nd), the lanes are added in a fixed order, so a token's
// scores do not depend on the tokens beside it.  Warp t then takes token t's softmax and choices.
template <typename T, int ROUTE_TOKENS>
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const T* __restrict__ h, int h_stride, const float* __restrict__ router, const float* __restrict__ correction,
                 int* __restrict__ ids, float* __restrict__ weights, int* __restrict__ counts, int tokens, int width,
                 int softmax_outputs, int experts, int top, float scale, int extra, float* __restrict__ extra_out,
                 int group_count, int group_keep, int renormalize) {
  extern __shared__ float smem[];
  int outputs = softmax_outputs + extra;              // rows of the router matrix
  float* zs = smem;                                   // ROUTE_TOKENS x outputs: scores
  float* choices = zs + ROUTE_TOKENS * outputs;       // ROUTE_TOKENS x outputs
  float* rows = smem + ((2 * ROUTE_TOKENS * outputs + 3) & ~3);   // ROUTE_TOKENS x width: the tokens' h as float32, on a 16-byte boundary
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t0 = blockIdx.x * ROUTE_TOKENS;
  const int here = min(ROUTE_TOKENS, tokens - t0);
  for (int i = threadIdx.x; i < ROUTE_TOKENS * width; i += ROUTE_THREADS) {
    const int r = i / width, k = i % width;
    rows[i] = r < here ? to_float(h[(size_t)(t0 + r) * h_stride + k]) : 0.f;
  }
  __syncthreads();
  for (int e = warp; e < outputs; e += ROUTE_THREADS / 32) {
    const float* w = router + (size_t)e * width;
    float dot[ROUTE_TOKENS];
#pragma unroll
    for (int r = 0; r < ROUTE_TOKENS; r++) dot[r] = 0.f;
    if ((width & 3) == 0) {
      // four weights a load; a lane's elements are added in ascending k, as in the scalar loop over its own elements
      for (int k = lane * 4; k < width; k += 128) {
        const float4 wk = *reinterpret_cast<const float4*>(w + k);
#pragma unroll
        for (int r = 0; r < ROUTE_TOKENS; r++) {
          const float4 xv = *reinterpret_cast<const float4*>(rows + r * width + k);
          dot[r] = fmaf(xv.x, wk.x, dot[r]);
          dot[r] = fmaf(xv.y, wk.y, dot[r]);
          dot[r] = fmaf(xv.z, wk.z, dot[r]);
          dot[r] = fmaf(xv.w, wk.w, dot[r]);
        }
      }
    } else {
      for (int k = lane; k < width; k += 32) {
        const float wk = w[k];
#pragma unroll
        for (int r = 0; r < ROUTE_TOKENS; r++) dot[r] = fmaf(rows[r * width + k], wk, dot[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < ROUTE_TOKENS; r++) {
      const float sum = warp_sum(dot[r]);
      if (lane == 0) zs[r * outputs + e] = sum;
    }
  }
  __syncthreads();
  if (warp >= here) return;
  const int t = t0 + warp;
  float* z = zs + warp * outputs;
  float* choice = choices + warp * outputs;
  for (int e = lane; e < extra; e += 32) extra_out[(size_t)t * extra + e] = z[softmax_outputs + e];
  outputs = softmax_outputs;                          // from here on: what the softmax is over
  float top_z = -INFINITY;
  for (int e = lane; e < outputs; e += 32) top_z = fmaxf(top_z, z[e]);
  top_z = warp_max(top_z);
  float sum = 0.f;
  for (int e = lane; e < outputs; e += 32) sum += expf(z[e] - top_z);
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < outputs; e += 32) {
    const float s = expf(z[e] - top_z) / sum;
    z[e] = s;
    choice[e] = s + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (group_count > 1 && group_keep < group_count) {
    // a group's score is its largest s; outputs outside the `group_keep` best groups (lowest index among equals) cannot
    // be taken.  A kept group is marked in its first output's choice.
    const int size = outputs / group_count;
    for (int kept = 0; kept < group_keep; kept++) {
      float best_s = -INFINITY;
      int best = 0x7fffffff;
      for (int g = lane; g < group_count; g += 32) {
        if (choice[g * size] == INFINITY) continue;          // already kept
        float top_s = -INFINITY;
        for (int e = g * size; e < (g + 1) * size; e++) top_s = fmaxf(top_s, z[e]);
        if (top_s > best_s) {
          best_s = top_s;
          best = g;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float other_s = __shfl_xor_sync(0xffffffffu, best_s, o);
        const int other = __shfl_xor_sync(0xffffffffu, best, o);
        if (other_s > best_s || (other_s == best_s && other < best)) {
          best_s = other_s;
          best = other;
        }
      }
      if (best >= group_count) break;
      __syncwarp();
      if (lane == 0) choice[best * size] = INFINITY;
      __syncwarp();
    }
    for (int g = lane; g < group_count; g += 32) {
      const bool kept = choice[g * size] == INFINITY;
      for (int e = g * size; e < (g + 1) * size; e++)
        choice[e] = kept ? z[e] + (correction ? correction[e] : 0.f) : -INFINITY;
    }
    __syncwarp();
  }
  // the largest choice `top` times; among equals the lowest index
  float taken = 0.f;
  for (int place = 0; place < top; place++) {
    float best_c = -INFINITY;
    int best = 0x7fffffff;
    for (int e = lane; e < outputs; e += 32)
      if (choice[e] > best_c) {
        best_c = choice[e];
        best = e;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other_c = __shfl_xor_sync(0xffffffffu, best_c, o);
      const int other = __shfl_xor_sync(0xffffffffu, best, o);
      if (other_c > best_c || (other_c == best_c && other < best)) {
        best_c = other_c;
        best = other;
      }
    }
    if (best >= outputs) best = 0;     // non-finite scores: the status of the logits will tell
    taken += z[best];
    if (lane == 0) {
      choice[best] = -INFINITY;
      ids[(size_t)t * top + place] = best;
      weights[(size_t)t * top + place] = z[best];
      if (best < experts) atomicAdd(&counts[best], 1);
    }
    __syncwarp();
  }
  const float norm = renormalize ? scale / (taken + 1e-20f) : scale;
  __syncwarp();
  for (int place = lane; place < top; place += 32) weights[(size_t)t * top + place] *= norm;
}

// One block.  counts -> offsets [experts + 1]; counts are left zeroed for the next call.
__global__ void __launch_bounds__(1024)
moe_arrange_kernel(const int* __restrict__ ids, int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ sorted,
                   int* __restrict__ place_of, int entries, int experts) {
  extern __shared__ int cursor[];       // experts
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; e++) {
      offsets[e] = at;
      cursor[e] = at;
      at += counts[e];
      counts[e] = 0;
    }
    offsets[experts] = at;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = ids[i];
    if (e < experts) {
      const int at = atomicAdd(&cursor[e], 1);
      sorted[at] = i;
      place_of[i] = at;
    } else {
      place_of[i] = -1;
    }
  }
}

__device__ __forceinline__ int expert_of(const int* offsets, int experts, int row) {
  int lo = 0, hi = experts;            // the last e with offsets[e] <= row
  while (hi - lo > 1) {
    const int mid = (lo + hi) / 2;
    if (offsets[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

// `limit` <= 0 names an expert without a gate: the exact gelu of its one product.
__device__ __forceinline__ float glu(float g, float u, float limit, float alpha) {
  if (limit <= 0.f) return 0.5f * g * (1.0f + erff(g * 0.7071067811865476f));
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
}

// grid (rows, column blocks); 8 warps, a warp per output column at a time.  w_gate_up [experts, 2 ff, width] with
// gate rows first; act [rows, ff].
template <typename T>
__global__ void __launch_bounds__(256)
moe_up_plain_kernel(const T* __restrict__ h, int h_stride, const int* __restrict__ sorted, const int* __restrict__ offsets,
                    const T* __restrict__ w_gate_up, T* __restrict__ act, int experts, int top, int width, int ff,
                    float limit, float alpha) {
  extern __shared__ float a[];          // width
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  if (row >= offsets[experts]) return;
  const int e = expert_of(offsets, experts, row);
  const T* src = h + (size_t)(sorted[row] / top) * h_stride;
  for (int k = threadIdx.x; k < width; k += blockDim.x) a[k] = to_float(src[k]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool gated = limit > 0.f;                      // else the matrix has ff rows per expert and no up rows
  const T* w = w_gate_up + (size_t)e * (gated ? 2 : 1) * ff * width;
  for (int j = blockIdx.y * 8 + warp; j < ff; j += gridDim.y * 8) {
    const T* wg = w + (size_t)j * width;
    const T* wu = w + (size_t)((gated ? ff : 0) + j) * width;
    float g = 0.f, u = 0.f;
    for (int k = lane; k < width; k += 32) {
      g = fmaf(a[k], to_float(wg[k]), g);
      if (gated) u = fmaf(a[k], to_float(wu[k]), u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    // the products' results are rounded to the activations' type before the activation, as separate products would leave them
    if (lane == 0) act[(size_t)row * ff + j] = from_float<T>(glu(to_float(from_float<T>(g)), to_float(from_float<T>(u)), limit, alpha));
  }
}

// w_down [experts, width, ff]; rows_out float32 [rows, width].
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_plain_kernel(const T* __restrict__ act, const int* __restrict__ offsets, const T* __restrict__ w_down,
                      float* __restrict__ rows_out, int experts, int width, int ff) {
  extern __shared__ float a[];          // ff
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  if (row >= offsets[experts]) return;
  const int e = expert_of(offsets, experts, row);
  for (int k = threadIdx.x; k < ff; k += blockDim.x) a[k] = to_float(act[(size_t)row * ff + k]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* w = w_down + (size_t)e * width * ff;
  for (int n = blockIdx.y * 8 + warp; n < width; n += gridDim.y * 8) {
    const T* wn = w + (size_t)n * ff;
    float s = 0.f;
    for (int k = lane; k < ff; k += 32) s = fmaf(a[k], to_float(wn[k]), s);
    s = warp_sum(s);
    if (lane == 0) rows_out[(size_t)row * width + n] = s;
  }
}


// ------------------------------------------------------------------------------------------ tensor cores
constexpr int GM = 128, GN = 128, GK = 64, GSTRIDE = GK + 8, GSTAGES = 3, GTHREADS = 256;
constexpr int GEMM_SMEM = GSTAGES * (GM + GN) * GSTRIDE * (int)sizeof(__nv_bfloat16);

// The CTA's tile: expert and first row, from the experts' offsets.  False: no such tile.
__device__ __forceinline__ bool find_tile(const int* offsets, int experts, int tile, int& expert, int& row0, int& row_end) {
  for (int e = 0; e < experts; e++) {
    const int begin = offsets[e], end = offsets[e + 1];
    const int tiles = (end - begin + GM - 1) / GM;
    if (tile < tiles) {
      expert = e;
      row0 = begin + tile * GM;
      row_end = end;
      return true;
    }
    tile -= tiles;
  }
  return false;
}

// UP: A rows are h[order[row] / top], B = w[expert] of [2 ff, K] (gate rows, then up rows), out = act [rows, ff] bfloat16.
// else: A rows are act[row] of [rows, K], B = w[expert] of [N, K], out = rows_out [rows, N] float32.
// KIND 0: the down product; 1: the gated up product (UP); 2: the up product of experts without a gate: A rows gathered
// like UP, B = w[expert] of [N, K], out = act [rows, N] bfloat16 = gelu(product), the exact form.
template <int KIND>
__global__ void __launch_bounds__(GTHREADS)
moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ a, int a_stride, const int* __restrict__ order,
                    const int* __restrict__ offsets, const __nv_bfloat16* __restrict__ w, void* __restrict__ out,
                    int experts, int top, int N, int K, float limit, float alpha) {
  extern __shared__ __align__(16) unsigned char gemm_smem[];
  typedef __nv_bfloat16 (*Tile)[GSTRIDE];
  __shared__ const __nv_bfloat16* a_rows[GM];
  pdl_launch_dependents();
  pdl_wait();
  constexpr bool UP = KIND == 1, GATHER = KIND != 0;
  int expert, row0, row_end;
  if (!find_tile(offsets, experts, blockIdx.x, expert, row0, row_end)) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = warp & 3, wn = warp >> 2;
  const int ff = UP ? N : 0;                         // UP: N is the experts' size, the matrix has 2 N rows
  const int n0 = blockIdx.y * (UP ? GN / 2 : GN);
  const __nv_bfloat16* wexp = w + (size_t)expert * (UP ? 2 * N : N) * K;
  if (tid < GM) {
    const int row = row0 + tid;
    a_rows[tid] = row < row_end ? (GATHER ? a + (size_t)(order[row] / top) * a_stride : a + (size_t)row * a_stride) : nullptr;
  }
  __syncthreads();
  auto As = [&](int stage) { return (Tile)(gemm_smem + (size_t)stage * (GM + GN) * GSTRIDE * sizeof(__nv_bfloat16)); };
  auto Ws = [&](int stage) { return (Tile)(gemm_smem + ((size_t)stage * (GM + GN) + GM) * GSTRIDE * sizeof(__nv_bfloat16)); };
  auto load = [&](int stage, int k0) {
    Tile at = As(stage), wt = Ws(stage);
#pragma unroll
    for (int i = 0; i < GM * (GK / 8) / GTHREADS; i++) {
      const int idx = tid + i * GTHREADS, row = idx / (GK / 8), c = (idx % (GK / 8)) * 8;
      const bool in_k = k0 + c < K;
      const __nv_bfloat16* src = a_rows[row];
      if (src && in_k) cp_async16(&at[row][c], src + k0 + c);
      else *(uint4*)&at[row][c] = make_uint4(0, 0, 0, 0);
      int wrow;                                       // the matrix row behind tile row `row`
      bool in_n;
      if (UP) {
        const int j = n0 + (row & 63);
        in_n = j < ff;
        wrow = (row < 64 ? 0 : ff) + j;
      } else {
        wrow = n0 + row;
        in_n = wrow < N;
      }
      if (in_n && in_k) cp_async16(&wt[row][c], wexp + (size_t)wrow * K + k0 + c);
      else *(uint4*)&wt[row][c] = make_uint4(0, 0, 0, 0);
    }
  };
  float acc[2][8][4];
#pragma unroll
  for (int mi = 0; mi < 2; mi++)
#pragma unroll
    for (int ni = 0; ni < 8; ni++) acc[mi][ni][0] = acc[mi][ni][1] = acc[mi][ni][2] = acc[mi][ni][3] = 0.f;
  const int steps = (K + GK - 1) / GK;
#pragma unroll
  for (int s = 0; s < GSTAGES - 1; s++) {
    if (s < steps) load(s, s * GK);
    cp_async_commit();
  }
  for (int t = 0; t < steps; t++) {
    cp_async_wait<GSTAGES - 2>();
    __syncthreads();
    if (t + GSTAGES - 1 < steps) load((t + GSTAGES - 1) % GSTAGES, (t + GSTAGES - 1) * GK);
    cp_async_commit();
    Tile at = As(t % GSTAGES), wt = Ws(t % GSTAGES);
#pragma unroll
    for (int kk = 0; kk < GK / 16; kk++) {
      uint32_t af[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; mi++)
        ldmatrix_x4(af[mi], &at[wm * 32 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int n2 = 0; n2 < 4; n2++) {
        // UP: the warp's 32 gate columns (tile rows wn * 32 ..) and the 32 up columns that go with them (64 + wn * 32 ..)
        const int base = UP ? (n2 < 2 ? wn * 32 + n2 * 16 : 64 + wn * 32 + (n2 - 2) * 16) : wn * 64 + n2 * 16;
        uint32_t b[4];
        ldmatrix_x4(b, &wt[base + (lane & 7) + (lane >> 4) * 8][kk * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
        for (int mi = 0; mi < 2; mi++) {
          mma_bf16(acc[mi][2 * n2], af[mi], b[0], b[1]);
          mma_bf16(acc[mi][2 * n2 + 1], af[mi], b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  const int gr = lane >> 2, qc = lane & 3;
#pragma unroll
  for (int mi = 0; mi < 2; mi++)
#pragma unroll
    for (int half = 0; half < 2; half++) {
      const int row = row0 + wm * 32 + mi * 16 + gr + half * 8;
      if (row >= row_end) continue;
      if (UP) {
        __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)row * ff;
#pragma unroll
        for (int ni = 0; ni < 4; ni++) {
          const int j = n0 + wn * 32 + ni * 8 + qc * 2;
          if (j >= ff) continue;
          float v[2];
#pragma unroll
          for (int c = 0; c < 2; c++) {
            // rounded to bfloat16 before the activation, as separate products would leave them
            const float g = __bfloat162float(__float2bfloat16_rn(acc[mi][ni][half * 2 + c]));
            const float u = __bfloat162float(__float2bfloat16_rn(acc[mi][ni + 4][half * 2 + c]));
            v[c] = glu(g, u, limit, alpha);
          }
          *(__nv_bfloat162*)(dst + j) = __floats2bfloat162_rn(v[0], v[1]);
        }
      } else if (KIND == 2) {
        __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)row * N;
#pragma unroll
        for (int ni = 0; ni < 8; ni++) {
          const int n = n0 + wn * 64 + ni * 8 + qc * 2;
          if (n >= N) continue;
          // rounded to bfloat16 before the activation, as a separate product would leave it
          const float g0 = __bfloat162float(__float2bfloat16_rn(acc[mi][ni][half * 2]));
          const float g1 = __bfloat162float(__float2bfloat16_rn(acc[mi][ni][half * 2 + 1]));
          *(__nv_bfloat162*)(dst + n) = __floats2bfloat162_rn(glu(g0, 0.f, 0.f, 0.f), glu(g1, 0.f, 0.f, 0.f));
        }
      } else {
        float* dst = (float*)out + (size_t)row * N;
#pragma unroll
        for (int ni = 0; ni < 8; ni++) {
          const int n = n0 + wn * 64 + ni * 8 + qc * 2;
          if (n < N) *(float2*)(dst + n) = make_float2(acc[mi][ni][half * 2], acc[mi][ni][half * 2 + 1]);
        }
      }
    }
}

// ------------------------------------------------------------------------------------------ a handful of tokens
// With at most FEW tokens in the step no expert has more than FEW rows.  A CTA takes (expert, block of output columns),
// keeps the expert's rows in shared memory and streams each weight row once with 16-byte loads for all of them: a warp
// per output column, eight elements a lane and step, float32 sums added across the lanes in a fixed order.
constexpr int FEW = 8, FEW_COLS = 32;

template <bool UP>
__global__ void __launch_bounds__(256)
moe_few_kernel(const __nv_bfloat16* __restrict__ a, int a_stride, const int* __restrict__ order, const int* __restrict__ offsets,
               const __nv_bfloat16* __restrict__ w, void* __restrict__ out, int top, int N, int K, float limit, float alpha) {
  extern __shared__ __align__(16) unsigned char few_smem[];
  __nv_bfloat16* rows = (__nv_bfloat16*)few_smem;            // FEW x K
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.x, row0 = offsets[e], count = min(offsets[e + 1] - row0, FEW);
  if (count <= 0) return;
  const int chunks = K / 8;
  for (int idx = threadIdx.x; idx < count * chunks; idx += blockDim.x) {
    const int r = idx / chunks, c = idx % chunks;
    const __nv_bfloat16* src = UP ? a + (size_t)(order[row0 + r] / top) * a_stride : a + (size_t)(row0 + r) * a_stride;
    *(uint4*)(rows + (size_t)r * K + c * 8) = *(const uint4*)(src + c * 8);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool gated = UP && limit > 0.f;               // else one matrix row per output
  const __nv_bfloat16* wexp = w + (size_t)e * (gated ? 2 * N : N) * K;
  for (int j = blockIdx.y * FEW_COLS + warp; j < min(N, (blockIdx.y + 1) * FEW_COLS); j += 8) {
    const __nv_bfloat16* w0 = wexp + (size_t)j * K;
    const __nv_bfloat16* w1 = wexp + (size_t)(N + j) * K;     // UP: the up row that goes with gate row j
    float s0[FEW], s1[FEW];
#pragma unroll
    for (int r = 0; r < FEW; r++) s0[r] = s1[r] = 0.f;
    for (int c = lane; c < chunks; c += 32) {
      const uint4 g = *(const uint4*)(w0 + c * 8);
      uint4 u = make_uint4(0, 0, 0, 0);
      if (gated) u = *(const uint4*)(w1 + c * 8);
      const __nv_bfloat162* gp = (const __nv_bfloat162*)&g;
      const __nv_bfloat162* up = (const __nv_bfloat162*)&u;
#pragma unroll
      for (int r = 0; r < FEW; r++) {
        if (r >= count) break;
        const uint4 x = *(const uint4*)(rows + (size_t)r * K + c * 8);
        const __nv_bfloat162* xp = (const __nv_bfloat162*)&x;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const float2 xv = __bfloat1622float2(xp[i]), gv = __bfloat1622float2(gp[i]);
          s0[r] = fmaf(xv.x, gv.x, s0[r]);
          s0[r] = fmaf(xv.y, gv.y, s0[r]);
          if (gated) {
            const float2 uv = __bfloat1622float2(up[i]);
            s1[r] = fmaf(xv.x, uv.x, s1[r]);
            s1[r] = fmaf(xv.y, uv.y, s1[r]);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < FEW; r++) {
      if (r >= count) break;
      const float g = warp_sum(s0[r]);
      if (UP) {
        const float u = gated ? warp_sum(s1[r]) : 0.f;
        if (lane == 0)
          ((__nv_bfloat16*)out)[(size_t)(row0 + r) * N + j] = __float2bfloat16_rn(
              glu(__bfloat162float(__float2bfloat16_rn(g)), __bfloat162float(__float2bfloat16_rn(u)), limit, alpha));
      } else if (lane == 0) {
        ((float*)out)[(size_t)(row0 + r) * N + j] = g;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ y, const T* __restrict__ h, int h_stride, const int* __restrict__ ids,
                   const float* __restrict__ weights, const int* __restrict__ place_of, const float* __restrict__ rows,
                   int width, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int n = threadIdx.x; n < width; n += blockDim.x) {
    float sum = 0.f;
    for (int place = 0; place < top; place++) {
      const int at = place_of[(size_t)t * top + place];
      const float w = weights[(size_t)t * top + place];
      sum = fmaf(w, at < 0 ? to_float(h[(size_t)t * h_stride + n]) : rows[(size_t)at * width + n], sum);
    }
    y[(size_t)t * width + n] += sum;
  }
}

// widths in multiples of 4: four columns a thread, the same sums in the same order
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_vec_kernel(float* __restrict__ y, const T* __restrict__ h, int h_stride, const float* __restrict__ weights,
                       const int* __restrict__ place_of, const float* __restrict__ rows, int width, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int n = threadIdx.x * 4; n < width; n += blockDim.x * 4) {
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int place = 0; place < top; place++) {
      const int at = place_of[(size_t)t * top + place];
      const float w = weights[(size_t)t * top + place];
      float4 v;
      if (at < 0) {
        const T* src = h + (size_t)t * h_stride + n;
        v = make_float4(to_float(src[0]), to_float(src[1]), to_float(src[2]), to_float(src[3]));
      } else {
        v = *(const float4*)(rows + (size_t)at * width + n);
      }
      sum.x = fmaf(w, v.x, sum.x); sum.y = fmaf(w, v.y, sum.y); sum.z = fmaf(w, v.z, sum.z); sum.w = fmaf(w, v.w, sum.w);
    }
    float4* dst = (float4*)(y + (size_t)t * width + n);
    float4 old = *dst;
    old.x += sum.x; old.y += sum.y; old.z += sum.z; old.w += sum.w;
    *dst = old;
  }
}

}  // namespace

// `outputs`: what the softmax is over; the router matrix has `outputs + extra` rows, and extra_out [tokens, extra] gets the
// last rows' products.  `correction` may be null (none).
SPROUT_API int sprout_moe_route(const void* h, int h_stride, int dtype, const float* router, const float* correction, int* ids,
                                float* weights, int* counts, int tokens, int width, int outputs, int experts, int top,
                                float scale, int extra, float* extra_out, int group_count, int group_keep, int renormalize,
                                cudaStream_t stream) {
  SPROUT_REQUIRE(h && router && ids && weights && counts, "moe_route: null pointer");
  SPROUT_REQUIRE(extra >= 0 && (extra == 0 || extra_out), "moe_route: the extra rows' products need a place");
  SPROUT_REQUIRE(group_count >= 1 && group_keep >= 1 && group_keep <= group_count && outputs % group_count == 0,
                 "moe_route: %d outputs do not form %d equal groups of which %d are kept", outputs, group_count, group_keep);
  SPROUT_REQUIRE(group_keep == group_count || top <= group_keep * (outputs / group_count),
                 "moe_route: the kept groups hold fewer outputs than are taken");
  SPROUT_REQUIRE(tokens > 0 && width > 0 && outputs > 0 && experts >= 0 && experts <= outputs && top > 0 && top <= outputs,
                 "moe_route: bad sizes (outputs %d, experts %d, top %d)", outputs, experts, top);
  const int rows_of_router = outputs + extra;
  const int per_block = tokens > 64 && ((size_t)8 * (2 * rows_of_router + width) + 4) * sizeof(float) <= 200 * 1024 ? 8 : 1;
  const size_t smem = ((size_t)per_block * (2 * rows_of_router + width) + 4) * sizeof(float);
  SPROUT_REQUIRE(smem <= 200 * 1024, "moe_route: too many router outputs (%d) or too wide rows (%d)", outputs, width);
  static bool prepared = false;
  if (!prepared) {
    cudaFuncSetAttribute(moe_route_kernel<float, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(moe_route_kernel<float, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    prepared = true;
  }
  dim3 grid((tokens + per_block - 1) / per_block);
#define ROUTE(T, N)                                                                                                    \
  sprout_launch(moe_route_kernel<T, N>, grid, dim3(ROUTE_THREADS), smem, stream, (const T*)h, h_stride, router, correction, ids, \
                weights, counts, tokens, width, outputs, experts, top, scale, extra, extra_out, group_count, group_keep, renormalize)
  if (dtype == SPROUT_F32) {
    if (per_block == 1) ROUTE(float, 1); else ROUTE(float, 8);
  } else if (dtype == SPROUT_BF16) {
    if (per_block == 1) ROUTE(__nv_bfloat16, 1); else ROUTE(__nv_bfloat16, 8);
  } else {
    return sprout_fail("moe_route: unknown dtype %d", dtype);
  }
#undef ROUTE
  return sprout_check_launch("moe_route");
}

SPROUT_API int sprout_moe_arrange(const int* ids, int* counts, int* offsets, int* sorted, int* place_of, int entries,
                                  int experts, cudaStream_t stream) {
  SPROUT_REQUIRE(ids && counts && offsets && sorted && place_of && entries > 0 && experts > 0 && experts <= 8192,
                 "moe_arrange: bad arguments");
  sprout_launch(moe_arrange_kernel, dim3(1), dim3(1024), (size_t)experts * sizeof(int), stream, ids, counts, offsets, sorted,
                place_of, entries, experts);
  return sprout_check_launch("moe_arrange");
}

SPROUT_API int sprout_moe_up_plain(const void* h, int h_stride, int dtype, const int* sorted, const int* offsets,
                                   const void* w_gate_up, void* act, int max_rows, int experts, int top, int width, int ff,
                                   float limit, float alpha, cudaStream_t stream) {
  SPROUT_REQUIRE(h && sorted && offsets && w_gate_up && act && max_rows > 0 && experts > 0 && width > 0 && ff > 0,
                 "moe_up: bad arguments");
  SPROUT_REQUIRE(width <= 12000, "moe_up: width up to 12000");
  dim3 grid(max_rows, ff >= 512 ? 4 : 1);
  const size_t smem = (size_t)width * sizeof(float);
  if (dtype == SPROUT_F32)
    sprout_launch(moe_up_plain_kernel<float>, grid, dim3(256), smem, stream, (const float*)h, h_stride, sorted, offsets,
                  (const float*)w_gate_up, (float*)act, experts, top, width, ff, limit, alpha);
  else if (dtype == SPROUT_BF16)
    sprout_launch(moe_up_plain_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)h, h_stride, sorted,
                  offsets, (const __nv_bfloat16*)w_gate_up, (__nv_bfloat16*)act, experts, top, width, ff, limit, alpha);
  else
    return sprout_fail("moe_up: unknown dtype %d", dtype);
  return sprout_check_launch("moe_up_plain");
}

SPROUT_API int sprout_moe_down_plain(const void* act, int dtype, const int* offsets, const void* w_down, float* rows_out,
                                     int max_rows, int experts, int width, int ff, cudaStream_t stream) {
  SPROUT_REQUIRE(act && offsets && w_down && rows_out && max_rows > 0 && experts > 0 && width > 0 && ff > 0,
                 "moe_down: bad arguments");
  SPROUT_REQUIRE(ff <= 12000, "moe_down: expert size up to 12000");
  dim3 grid(max_rows, width >= 512 ? 4 : 1);
  const size_t smem = (size_t)ff * sizeof(float);
  if (dtype == SPROUT_F32)
    sprout_launch(moe_down_plain_kernel<float>, grid, dim3(256), smem, stream, (const float*)act, offsets,
                  (const float*)w_down, rows_out, experts, width, ff);
  else if (dtype == SPROUT_BF16)
    sprout_launch(moe_down_plain_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)act, offsets,
                  (const __nv_bfloat16*)w_down, rows_out, experts, width, ff);
  else
    return sprout_fail("moe_down: unknown dtype %d", dtype);
  return sprout_check_launch("moe_down_plain");
}

// Whether the tensor-core products take these sizes: rows of 16-byte multiples, pairs of outputs.
SPROUT_API int sprout_moe_mma_supported(int width, int ff, int h_stride) {
  return width % 8 == 0 && ff % 8 == 0 && h_stride % 8 == 0;
}

// act [entries, ff] bfloat16 = glu(W_gate a, W_up a); rows_out [entries, width] float32 = W_down act, over the arranged rows.
SPROUT_API int sprout_moe_experts_mma(const void* h, int h_stride, const int* order, const int* offsets, const void* w_gate_up,
                                      const void* w_down, void* act, float* rows_out, int entries, int experts, int top,
                                      int width, int ff, float limit, float alpha, cudaStream_t stream) {
  SPROUT_REQUIRE(h && order && offsets && w_gate_up && w_down && act && rows_out, "moe_experts_mma: null pointer");
  SPROUT_REQUIRE(entries > 0 && experts > 0 && top > 0 && sprout_moe_mma_supported(width, ff, h_stride),
                 "moe_experts_mma: sizes must be multiples of 8 (width %d, ff %d, row stride %d)", width, ff, h_stride);
  SPROUT_REQUIRE((((uintptr_t)h | (uintptr_t)w_gate_up | (uintptr_t)w_down | (uintptr_t)act | (uintptr_t)rows_out) & 15) == 0,
                 "moe_experts_mma: buffers must start on 16-byte boundaries");
  if (entries <= FEW * top && (size_t)FEW * (width > ff ? width : ff) * 2 <= 160 * 1024) {
    // at most FEW tokens: no expert has more rows than that, and the products are streams of weights
    static bool few_prepared = false;
    if (!few_prepared) {
      cudaFuncSetAttribute(moe_few_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      cudaFuncSetAttribute(moe_few_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      few_prepared = true;
    }
    sprout_launch(moe_few_kernel<true>, dim3(experts, (ff + FEW_COLS - 1) / FEW_COLS), dim3(256), (size_t)FEW * width * 2, stream,
                  (const __nv_bfloat16*)h, h_stride, order, offsets, (const __nv_bfloat16*)w_gate_up, act, top, ff, width, limit, alpha);
    if (int code = sprout_check_launch("moe_up_few")) return code;
    sprout_launch(moe_few_kernel<false>, dim3(experts, (width + FEW_COLS - 1) / FEW_COLS), dim3(256), (size_t)FEW * ff * 2, stream,
                  (const __nv_bfloat16*)act, ff, order, offsets, (const __nv_bfloat16*)w_down, (void*)rows_out, top, width, ff, 0.f, 0.f);
    return sprout_check_launch("moe_down_few");
  }
  static bool prepared = false;
  if (!prepared) {
    cudaFuncSetAttribute(moe_gemm_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(moe_gemm_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    cudaFuncSetAttribute(moe_gemm_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    prepared = true;
  }
  const int tiles = (entries + GM - 1) / GM + experts;       // at most this many row tiles, whatever the routing
  if (limit > 0.f)
    sprout_launch(moe_gemm_mma_kernel<1>, dim3(tiles, (ff + GN / 2 - 1) / (GN / 2)), dim3(GTHREADS), GEMM_SMEM, stream,
                  (const __nv_bfloat16*)h, h_stride, order, offsets, (const __nv_bfloat16*)w_gate_up, act, experts, top, ff, width,
                  limit, alpha);
  else
    sprout_launch(moe_gemm_mma_kernel<2>, dim3(tiles, (ff + GN - 1) / GN), dim3(GTHREADS), GEMM_SMEM, stream,
                  (const __nv_bfloat16*)h, h_stride, order, offsets, (const __nv_bfloat16*)w_gate_up, act, experts, top, ff, width,
                  limit, alpha);
  if (int code = sprout_check_launch("moe_up_mma")) return code;
  sprout_launch(moe_gemm_mma_kernel<0>, dim3(tiles, (width + GN - 1) / GN), dim3(GTHREADS), GEMM_SMEM, stream,
                (const __nv_bfloat16*)act, ff, order, offsets, (const __nv_bfloat16*)w_down, (void*)rows_out, experts, top, width, ff,
                0.f, 0.f);
  return sprout_check_launch("moe_down_mma");
}

SPROUT_API int sprout_moe_combine(float* y, const void* h, int h_stride, int dtype, const int* ids, const float* weights,
                                  const int* place_of, const float* rows, int tokens, int width, int top,
                                  cudaStream_t stream) {
  SPROUT_REQUIRE(y && h && ids && weights && place_of && tokens > 0 && width > 0 && top > 0, "moe_combine: bad arguments");
  const bool vec = width % 4 == 0 && (((uintptr_t)y | (uintptr_t)rows) & 15) == 0;
  if (vec && dtype == SPROUT_F32)
    sprout_launch(moe_combine_vec_kernel<float>, dim3(tokens), dim3(256), 0, stream, y, (const float*)h, h_stride, weights, place_of,
                  rows, width, top);
  else if (vec && dtype == SPROUT_BF16)
    sprout_launch(moe_combine_vec_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, y, (const __nv_bfloat16*)h, h_stride,
                  weights, place_of, rows, width, top);
  else if (dtype == SPROUT_F32)
    sprout_launch(moe_combine_kernel<float>, dim3(tokens), dim3(256), 0, stream, y, (const float*)h, h_stride, ids, weights,
                  place_of, rows, width, top);
  else if (dtype == SPROUT_BF16)
    sprout_launch(moe_combine_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, y, (const __nv_bfloat16*)h, h_stride,
                  ids, weights, place_of, rows, width, top);
  else
    return sprout_fail("moe_combine: unknown dtype %d", dtype);
  return sprout_check_launch("moe_combine");
}
