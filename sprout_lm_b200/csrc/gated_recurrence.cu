// Recurrent mixers whose decay comes from the input, and the row kernels around them.  All arithmetic is float32;
// the element type of the projections (float or bfloat16) is a template parameter.
//
//  * gated_scan:   per request and head, token by token:
//                      S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T,   o_t = S_t^T (q_scale q_t) + skip_h v_t
//                  with S [dim, vdim] float32 in the request's state slot.  Two ways to make a_t and c_t:
//                    per key channel (gated linear attention): a_t[i] = sigmoid(z_t[i] + bias[i])^(1/tau), c_t = 1;
//                    per head (a selective state space):      dt = softplus(z_t[h] + bias[h]), a_t[i] = exp(-exp(a_log[h]) dt),
//                                                             c_t = dt;
//                    given (a matrix memory with exponential gates): a_t and c_t per head come ready-made from the
//                                                             caller (`da`, `dc`), whatever the portion's length.
//                  With `ones_col` the value row gets one more column that is always 1 (column `v_cols` of the state
//                  and of the output): the state's extra column is then sum of the decayed c_t k_t, a normaliser.
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

enum ScanDecay : int { DECAY_PER_CHANNEL = 0, DECAY_PER_HEAD = 1, DECAY_GIVEN = 2 };

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
  // portions cut into chunks (null / 0 when every request's tokens are walked by one block):
  const float* da;                     // decays made beforehand: [tokens, heads * dim] per channel, [tokens, heads] per head
  const float* dc;                     // per head: the factor on k, [tokens, heads]
  float* sums;                         // [max_chunks, heads, dim, vdim]: a chunk's own sums, then the state before the chunk
  float* prods;                        // [max_chunks, heads, dim]: the product of a chunk's decays
  int chunk, requests;
  int v_cols, ones_col;                // columns the value rows really have (<= vdim); column v_cols of the state is fed 1
};

// The chunks of all requests are numbered in the requests' order, ceil(tokens / chunk) each.  Finds chunk `index`:
// its request, its place among the request's chunks and how many the request has; false beyond the last chunk.
__device__ __forceinline__ bool find_chunk(const int* q_start, int requests, int chunk, int index, int& r, int& c, int& n) {
  for (int i = 0; i < requests; i++) {
    n = (q_start[i + 1] - q_start[i] + chunk - 1) / chunk;
    if (index < n) { r = i; c = index; return true; }
    index -= n;
  }
  return false;
}

enum ScanPhase : int { SCAN_WHOLE = 0, SCAN_CHUNK_SUMS = 1, SCAN_CHUNK_OUT = 2 };

constexpr int SCAN_THREADS = 128, SCAN_MAX_TOKENS = 8;

// A block of SCAN_THREADS threads owns (request, head, `cb` value columns).  A thread keeps a tile of ROWS x COLS
// elements of the state in registers from the first token to the last: the state's rows are dealt to `slices` lanes
// of a warp (a power of two; the thread of slice s has rows s, s + slices, s + 2 slices, ...), the columns in groups of
// COLS to the threads of equal slice, so every (q, k, a) triple read from shared memory serves COLS columns.
// Tokens come `batch` at a time: while the threads walk a batch's tokens over their registers, the next batch's q, k,
// decay inputs and values are on their way from memory into registers; at the batch's end they are turned into
// float32 vectors in shared memory ([q_scale q | c k | a] per row).  The slices of a column add their parts of o with
// shuffles.  Each element of S sees S <- fma(a, S, (c k) v) once per token in the tokens' order, so the result does not
// depend on the cutting or on the batch.
//
// Long portions are cut into chunks of `p.chunk` tokens so that more blocks than (request, head, columns) have work, in
// three launches: SCAN_CHUNK_SUMS walks every chunk but a request's last from a zero state and leaves the chunk's own
// sums and the product of its decays; scan_carry_kernel turns them, in the chunks' order, into the state before each
// chunk; SCAN_CHUNK_OUT walks every chunk from that state, writes the outputs, and the last chunk writes the
// request's state.  The decays of these two walks are made beforehand by scan_decay_kernel (each is needed by all
// blocks of columns and in both walks).  Against the single walk only the association of the decays' products
// differs: (a_n ... a_1) S + sums instead of a_n (... (a_1 S)).
template <typename T, int ROWS, int COLS, int PHASE>
__global__ void __launch_bounds__(SCAN_THREADS, ROWS == 8 ? 4 : 2)
gated_scan_kernel(const ScanParams<T> p, int slices_log2, int batch) {
  constexpr int ROWS_LOG2 = ROWS == 8 ? 3 : 5;
  static_assert(ROWS == 8 || ROWS == 32, "rows of a thread's tile");
  constexpr int EPT = ROWS == 8 ? 8 : 16;            // row vectors a thread fetches per batch: batch * slices * ROWS / threads
  constexpr int VPT = SCAN_MAX_TOKENS;               // values a thread fetches per batch: batch * cb / threads
  extern __shared__ float4 scan_smem[];
  const int slices = 1 << slices_log2, dim = p.dim;
  const int rows_log2 = slices_log2 + ROWS_LOG2, rows_pad = 1 << rows_log2;
  const int cb_log2 = 7 - slices_log2 + (COLS == 4 ? 2 : 0), cb = 1 << cb_log2;
  static_assert(COLS == 1 || COLS == 4, "columns of a thread's tile");
  float4* tok = scan_smem;                                             // [batch][rows_pad]: (q, k, a, -)
  float* vt = reinterpret_cast<float*>(tok + (size_t)batch * rows_pad);  // [batch][cb]
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.y, tid = threadIdx.x;
  int r = blockIdx.x, chunk_at = 0, chunk_count = 1;
  if (PHASE != SCAN_WHOLE && p.sums != nullptr) {      // without scratch every request is one chunk: block x walks request x
    if (!find_chunk(p.q_start, p.requests, p.chunk, blockIdx.x, r, chunk_at, chunk_count)) return;
    if (PHASE == SCAN_CHUNK_SUMS && chunk_at == chunk_count - 1) return;      // nothing comes after it
  }
  const bool last_chunk = chunk_at == chunk_count - 1;
  const int slice = tid & (slices - 1), col_local = (tid >> slices_log2) * COLS;
  const int col = blockIdx.z * cb + col_local;                          // the first of the thread's columns
  const int slot = p.state_slots[r];
  if (slot < 0 || slot >= p.num_slots) {
    if (tid == 0) atomicOr(p.status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  const int g = h / (p.heads / p.groups);
  const bool per_head = p.mode != DECAY_PER_CHANNEL;
  float* mine = p.state + (((size_t)slot * p.heads + h) * dim) * p.vdim;
  // the chunk's place in the scratch: the blocks before it belong to the requests before r and to r's earlier chunks
  float* held = PHASE == SCAN_WHOLE ? nullptr : p.sums + (((size_t)(blockIdx.x) * p.heads + h) * dim) * p.vdim;
  const float* from = (PHASE == SCAN_WHOLE || chunk_count == 1) ? mine : held;
  const bool vectors = (p.vdim & 3) == 0;             // rows of the state start on 16-byte boundaries
  float S[ROWS][COLS], P[PHASE == SCAN_CHUNK_SUMS ? ROWS : 1];
#pragma unroll
  for (int j = 0; j < ROWS; j++) {
    const int row = j * slices + slice;
    if (COLS == 4 && vectors) {                       // four columns of a row in one access
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (PHASE != SCAN_CHUNK_SUMS && col < p.vdim && row < dim) x = *reinterpret_cast<const float4*>(from + (size_t)row * p.vdim + col);
      S[j][0] = x.x; S[j][1 % COLS] = x.y; S[j][2 % COLS] = x.z; S[j][3 % COLS] = x.w;
    } else {
#pragma unroll
      for (int c = 0; c < COLS; c++)
        S[j][c] = (PHASE != SCAN_CHUNK_SUMS && col + c < p.vdim && row < dim) ? from[(size_t)row * p.vdim + col + c] : 0.f;
    }
    if (PHASE == SCAN_CHUNK_SUMS) P[j] = 1.f;
  }
  const float skip = p.skip ? p.skip[h] : 0.f;
  const float rate = p.mode == DECAY_PER_HEAD ? expf(p.a_log[h]) : 0.f;
  const int first = p.q_start[r] + chunk_at * (PHASE == SCAN_WHOLE ? 0 : p.chunk);
  const int last = PHASE == SCAN_WHOLE ? p.q_start[r + 1] : min(p.q_start[r + 1], first + p.chunk);
  auto z_at = [&](size_t index) { return p.z_f32 ? ((const float*)p.z)[index] : to_float(((const T*)p.z)[index]); };

  float rq[EPT], rk[EPT], rz[EPT], rc[PHASE == SCAN_WHOLE ? 1 : EPT], rv[VPT];
  auto fetch = [&](int t0) {                          // loads only: nothing waits for them here
    const int n = min(batch, last - t0);
    // the batch's first rows once in 64-bit; within the batch 32-bit offsets do (at most SCAN_MAX_TOKENS rows further)
    const size_t tb = (size_t)t0;
    const T* qrow = p.q + tb * p.q_stride + (size_t)g * dim;
    const T* krow = p.k + tb * p.k_stride + (size_t)g * dim;
    const T* vrow = p.v + tb * p.v_stride + (size_t)h * p.v_cols;
    const float* arow = PHASE == SCAN_WHOLE ? nullptr : p.da + (per_head ? tb * p.heads + h : (tb * p.heads + h) * dim);
    const float* crow = (PHASE == SCAN_WHOLE || !per_head) ? nullptr : p.dc + tb * p.heads + h;
#pragma unroll
    for (int u = 0; u < EPT; u++) {
      const int e = tid + u * SCAN_THREADS, tt = e >> rows_log2, i = e & (rows_pad - 1);
      rq[u] = rk[u] = rz[u] = 0.f;
      if (PHASE != SCAN_WHOLE) rc[u] = 0.f;
      if (tt < n && i < dim) {
        if (PHASE != SCAN_CHUNK_SUMS) rq[u] = to_float(qrow[tt * p.q_stride + i]);
        rk[u] = to_float(krow[tt * p.k_stride + i]);
        if (PHASE == SCAN_WHOLE) {
          const size_t t = tb + tt;
          rz[u] = per_head ? z_at(t * p.z_stride + h) : z_at(t * p.z_stride + (size_t)h * dim + i);
        } else {
          rz[u] = per_head ? arow[tt * p.heads] : arow[tt * p.heads * dim + i];
          rc[u] = per_head ? crow[tt * p.heads] : 1.f;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < VPT; u++) {
      const int e = tid + u * SCAN_THREADS, tt = e >> cb_log2, column = blockIdx.z * cb + (e & (cb - 1));
      rv[u] = (tt < n && column < p.v_cols) ? to_float(vrow[tt * p.v_stride + column]) : (p.ones_col && tt < n && column == p.v_cols) ? 1.f : 0.f;
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
        if (PHASE != SCAN_WHOLE) {
          step = rc[u];
          decay = rz[u];
        } else if (per_head) {
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
    float* out_rows = p.out + (size_t)t0 * p.heads * p.vdim + (size_t)h * p.vdim + col;
    for (int tt = 0; tt < n; tt++) {
      float v[COLS], o[COLS];
      if (COLS == 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(vt + (tt << cb_log2) + col_local);
        v[0] = v4.x; v[1 % COLS] = v4.y; v[2 % COLS] = v4.z; v[3 % COLS] = v4.w;
      } else {
#pragma unroll
        for (int c = 0; c < COLS; c++) v[c] = vt[(tt << cb_log2) + col_local + c];
      }
#pragma unroll
      for (int c = 0; c < COLS; c++) o[c] = 0.f;
      const float4* cur = tok + ((size_t)tt << rows_log2) + slice;
#pragma unroll
      for (int j = 0; j < ROWS; j++) {
        const float4 x = cur[j << slices_log2];
#pragma unroll
        for (int c = 0; c < COLS; c++) {
          const float s = fmaf(x.z, S[j][c], x.y * v[c]);
          S[j][c] = s;
          if (PHASE != SCAN_CHUNK_SUMS) o[c] = fmaf(s, x.x, o[c]);
        }
        if (PHASE == SCAN_CHUNK_SUMS) P[j] *= x.z;
      }
      if (PHASE == SCAN_CHUNK_SUMS) continue;
      float* dst = out_rows + tt * p.heads * p.vdim;
      if (COLS == 4 && slices_log2 >= 2) {
        // four sums over the slices with five shuffles instead of four per sum: neighbours split the columns between
        // them (the even lane takes 0 and 1, the odd one 2 and 3), then pairs two apart split again; lane (b0, b1)
        // ends with column 2 b0 + b1, added up over the remaining lanes as usual
        const bool odd = slice & 1, upper = slice & 2;
        float keep0 = odd ? o[2 % COLS] : o[0], keep1 = odd ? o[3 % COLS] : o[1 % COLS];
        keep0 += __shfl_xor_sync(0xffffffffu, odd ? o[0] : o[2 % COLS], 1);
        keep1 += __shfl_xor_sync(0xffffffffu, odd ? o[1 % COLS] : o[3 % COLS], 1);
        float keep = upper ? keep1 : keep0;
        keep += __shfl_xor_sync(0xffffffffu, upper ? keep0 : keep1, 2);
        for (int d = 4; d < slices; d <<= 1) keep += __shfl_xor_sync(0xffffffffu, keep, d);
        const int c = 2 * (slice & 1) + ((slice >> 1) & 1);
        const float vc = c == 0 ? v[0] : c == 1 ? v[1 % COLS] : c == 2 ? v[2 % COLS] : v[3 % COLS];
        if (slice < 4 && col + c < p.vdim) dst[c] = fmaf(skip, vc, keep);
      } else {
#pragma unroll
        for (int c = 0; c < COLS; c++) {
          for (int d = slices >> 1; d > 0; d >>= 1) o[c] += __shfl_xor_sync(0xffffffffu, o[c], d);
          if (slice == 0 && col + c < p.vdim) dst[c] = fmaf(skip, v[c], o[c]);
        }
      }
    }
  }
  if (PHASE == SCAN_CHUNK_OUT && !last_chunk) return;
  float* to = PHASE == SCAN_CHUNK_SUMS ? held : mine;
#pragma unroll
  for (int j = 0; j < ROWS; j++) {
    const int row = j * slices + slice;
    if (COLS == 4 && vectors) {
      if (col < p.vdim && row < dim)
        *reinterpret_cast<float4*>(to + (size_t)row * p.vdim + col) = make_float4(S[j][0], S[j][1 % COLS], S[j][2 % COLS], S[j][3 % COLS]);
    } else {
#pragma unroll
      for (int c = 0; c < COLS; c++)
        if (col + c < p.vdim && row < dim) to[(size_t)row * p.vdim + col + c] = S[j][c];
    }
    if (PHASE == SCAN_CHUNK_SUMS && blockIdx.z == 0 && col_local == 0 && row < dim)
      p.prods[((size_t)blockIdx.x * p.heads + h) * dim + row] = P[j];
  }
}

// The decays of every token of the step, once: per key channel a = sigmoid(z + bias)^(1 / tau); per head
// dt = softplus(z + bias), a = exp(-exp(a_log) dt), c = dt.
__global__ void scan_decay_kernel(const void* __restrict__ z, int z_stride, int z_f32, int is_bf16, const float* __restrict__ bias,
                                  const float* __restrict__ a_log, float inv_tau, int mode, int heads, int dim, long long count,
                                  float* __restrict__ da, float* __restrict__ dc) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_token = mode == DECAY_PER_HEAD ? heads : heads * dim;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / per_token;
    const int c = (int)(e - t * per_token);
    const size_t at = (size_t)t * z_stride + c;
    const float zv = (z_f32 || !is_bf16) ? ((const float*)z)[at] : to_float(((const __nv_bfloat16*)z)[at]);
    if (mode == DECAY_PER_HEAD) {
      const float step = softplus_f(zv + bias[c]);
      da[e] = expf(-expf(a_log[c]) * step);
      dc[e] = step;
    } else {
      da[e] = expf(-softplus_f(-(zv + bias[c])) * inv_tau);
    }
  }
}

// In the chunks' order, per element of a request's state: the scratch's entry of chunk c (the chunk's own sums)
// becomes the state before chunk c; requests of one chunk are left alone (their walk starts from the state slot).
__global__ void scan_carry_kernel(float* __restrict__ sums, const float* __restrict__ prods, const float* __restrict__ state,
                                  const int* __restrict__ q_start, const int* __restrict__ state_slots, int num_slots, int chunk,
                                  int heads, int dim, int vdim) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.z, h = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = (q_start[r + 1] - q_start[r] + chunk - 1) / chunk;
  const int slot = state_slots[r];
  if (n < 2 || e >= dim * vdim || slot < 0 || slot >= num_slots) return;
  int base = 0;
  for (int i = 0; i < r; i++) base += (q_start[i + 1] - q_start[i] + chunk - 1) / chunk;
  const int row = e / vdim;
  const size_t per = (size_t)heads * dim * vdim;
  float* mine = sums + (size_t)base * per + (size_t)h * dim * vdim + e;
  const float* decays = prods + ((size_t)base * heads + h) * dim + row;
  float S = state[((size_t)slot * heads + h) * dim * vdim + e];
  const size_t decay_step = (size_t)heads * dim;
  for (int c0 = 0; c0 + 1 < n; c0 += 8) {              // eight chunks' loads are in flight before the first is used
    float own[8], a[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const bool there = c0 + u + 1 < n;
      own[u] = there ? mine[(size_t)(c0 + u) * per] : 0.f;
      a[u] = there ? decays[(size_t)(c0 + u) * decay_step] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      if (c0 + u + 1 >= n) break;
      mine[(size_t)(c0 + u) * per] = S;
      S = fmaf(a[u], S, own[u]);
    }
  }
  mine[(size_t)(n - 1) * per] = S;
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

template <typename T, int ROWS, int COLS>
int launch_scan_tiles(const ScanParams<T>& p, int requests, int max_chunks, cudaStream_t stream) {
  int slices_log2 = 0;
  while ((ROWS << slices_log2) < p.dim) slices_log2++;
  SPROUT_REQUIRE(slices_log2 <= 5, "gated_scan: key vectors too long (%d)", p.dim);
  const int slices = 1 << slices_log2, cb = SCAN_THREADS / slices * COLS;
  // tokens of a batch: what a thread stages in registers bounds it (row vectors: ROWS * slices * batch / threads <= 8 or 16;
  // values: cb * batch / threads <= SCAN_MAX_TOKENS)
  int batch = SCAN_MAX_TOKENS;
  const int by_rows = (ROWS == 8 ? 128 : 64) / slices, by_values = SCAN_MAX_TOKENS * slices / COLS;
  if (batch > by_rows) batch = by_rows;
  if (batch > by_values) batch = by_values;
  const size_t smem = (size_t)batch * ((size_t)ROWS * slices * sizeof(float4) + (size_t)cb * sizeof(float));
  const dim3 grid(requests, p.heads, (p.vdim + cb - 1) / cb);
  SPROUT_REQUIRE(grid.z <= 65535, "gated_scan: too many value columns");
  if (p.sums == nullptr && p.mode == DECAY_GIVEN) {
    sprout_launch(gated_scan_kernel<T, ROWS, COLS, SCAN_CHUNK_OUT>, grid, dim3(SCAN_THREADS), smem, stream, p, slices_log2, batch);
    return sprout_check_launch("gated_scan");
  }
  if (p.sums == nullptr) {
    sprout_launch(gated_scan_kernel<T, ROWS, COLS, SCAN_WHOLE>, grid, dim3(SCAN_THREADS), smem, stream, p, slices_log2, batch);
    return sprout_check_launch("gated_scan");
  }
  // `max_chunks` blocks per (head, columns): the chunks of all requests, found by their number
  const dim3 chunks(max_chunks, p.heads, grid.z);
  sprout_launch(gated_scan_kernel<T, ROWS, COLS, SCAN_CHUNK_SUMS>, chunks, dim3(SCAN_THREADS), smem, stream, p, slices_log2, batch);
  if (int rc = sprout_check_launch("gated_scan (chunk sums)")) return rc;
  SPROUT_REQUIRE(requests <= 65535, "gated_scan: too many requests");
  sprout_launch(scan_carry_kernel, dim3((p.dim * p.vdim + 255) / 256, p.heads, requests), dim3(256), 0, stream, p.sums,
                (const float*)p.prods, (const float*)p.state, p.q_start, p.state_slots, p.num_slots, p.chunk, p.heads, p.dim, p.vdim);
  if (int rc = sprout_check_launch("gated_scan (carry)")) return rc;
  sprout_launch(gated_scan_kernel<T, ROWS, COLS, SCAN_CHUNK_OUT>, chunks, dim3(SCAN_THREADS), smem, stream, p, slices_log2, batch);
  return sprout_check_launch("gated_scan (chunk outputs)");
}

template <typename T>
int launch_scan(const ScanParams<T>& p, int requests, int max_chunks, cudaStream_t stream) {
  // a thread's tile of the state: 8 rows x 4 columns up to 256 key channels, 32 rows of one column up to 1024
  if (p.dim <= 8 * 32) return launch_scan_tiles<T, 8, 4>(p, requests, max_chunks, stream);
  return launch_scan_tiles<T, 32, 1>(p, requests, max_chunks, stream);
}

}  // namespace

SPROUT_API int sprout_gated_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                                 const void* z, int z_stride, int z_f32, int dtype, const float* bias, const float* a_log, const float* skip,
                                 float inv_tau, float q_scale, int mode, int requests, int heads, int groups, int dim, int vdim,
                                 const int* q_start, const int* state_slots, float* state, int num_slots, float* out, int* status,
                                 int tokens, int chunk, int max_chunks, float* da, float* dc, float* sums, float* prods,
                                 int v_cols, int ones_col, cudaStream_t stream) {
  SPROUT_REQUIRE(q && k && v && q_start && state_slots && state && out && status, "gated_scan: null pointer");
  SPROUT_REQUIRE(mode == DECAY_GIVEN ? (da && dc) : (z && bias), "gated_scan: the decay's inputs are missing");
  SPROUT_REQUIRE(v_cols > 0 && v_cols <= vdim && (!ones_col || v_cols < vdim), "gated_scan: the value rows' columns do not fit the state's");
  if (mode == DECAY_GIVEN && !sums) {
    // one walk per request over ready-made decays: the outputs' walk of the chunked form with a chunk that holds any portion
    chunk = 1 << 30;
    max_chunks = requests;
  }
  if (sums && mode != DECAY_GIVEN) {
    // portions in chunks: scratch for the decays of every token and for every chunk's sums and decay product
    SPROUT_REQUIRE(chunk > 0 && max_chunks > 0 && tokens > 0 && da && prods && (mode != DECAY_PER_HEAD || dc),
                   "gated_scan: the chunked form needs its scratch");
    const long long count = (long long)tokens * (mode == DECAY_PER_HEAD ? heads : heads * dim);
    const long long blocks = (count + 255) / 256;
    sprout_launch(scan_decay_kernel, dim3((unsigned)(blocks < 148 * 16 ? blocks : 148 * 16)), dim3(256), 0, stream, z, z_stride, z_f32,
                  dtype == SPROUT_BF16 ? 1 : 0, bias, a_log, inv_tau, mode, heads, dim, count, da, dc);
    if (int rc = sprout_check_launch("gated_scan (decays)")) return rc;
  }
  SPROUT_REQUIRE(requests > 0 && heads > 0 && groups > 0 && heads % groups == 0 && dim > 0 && vdim > 0 && num_slots > 0,
                 "gated_scan: bad sizes");
  SPROUT_REQUIRE(mode == DECAY_PER_CHANNEL || (mode == DECAY_PER_HEAD && a_log) || mode == DECAY_GIVEN, "gated_scan: unknown decay form");
  SPROUT_REQUIRE(heads <= 65535, "gated_scan: too many heads");
  if (dtype == SPROUT_F32) {
    ScanParams<float> p{(const float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, z, z_stride, z_f32,
                        bias, a_log, skip, inv_tau, q_scale, mode, heads, groups, dim, vdim, q_start, state_slots, state,
                        num_slots, out, status, da, dc, sums, prods, chunk, requests, v_cols, ones_col};
    return launch_scan(p, requests, max_chunks, stream);
  }
  if (dtype == SPROUT_BF16) {
    ScanParams<__nv_bfloat16> p{(const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v,
                                v_stride, z, z_stride, z_f32, bias, a_log, skip, inv_tau, q_scale, mode, heads,
                                groups, dim, vdim, q_start, state_slots, state, num_slots, out, status, da, dc, sums, prods, chunk,
                                requests, v_cols, ones_col};
    return launch_scan(p, requests, max_chunks, stream);
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
