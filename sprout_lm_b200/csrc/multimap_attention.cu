// Attention whose heads hold one or two score maps over shared values (differential attention), on the
// paged cache, float32 arithmetic.
//
// A key/value head's cache row holds `maps` key vectors of `dim` elements side by side
// ([pages, kv_heads, page_tokens, maps * dim]); its value row has `vdim` elements
// ([pages, kv_heads, page_tokens, vdim]).  A query head has `maps` query vectors; map m of query head h
// scores against map m of key/value head h / (heads / kv_heads): score = scale * q . k, causal, softmax
// per map, a_m = softmax_m V.  The head's output is a_0 - lambda * a_1 (a_0 alone with one map), then,
// with `norm_eps` > 0, divided by its root mean square over vdim, and times `out_scale`.
//
//  * rope_maps_append:          rotates the first `rot` elements of every query and key vector by the
//                               token's position (half-split pairs) and appends keys and values to the cache; before
//                               the rotation it can divide every vector by its root mean square and multiply it by a
//                               weight (one for queries, one for keys).
// Options of both attention kernels: a mask (a window, a window that also keeps the first positions, chunks), a cap on
// the scaled scores (cap * tanh(score / cap)), a sink per head in the softmax denominator, a gate per head.
//  * multimap_attention_simple: one block per (token, query head); keys in chunks of 128 aligned to
//                               absolute position with running maxima and sums: what is done for a query
//                               does not depend on how the tokens were cut into steps.
//  * multimap_attention_mma:    bfloat16 on tensor cores (`mma.sync.m16n8k16`): a CTA of 4 warps owns 64
//                               (token, head of one key/value group) rows of a request and walks the keys in
//                               tiles of 64 through a double-buffered cp.async ring; a warp holds both maps of
//                               its 16 rows (scores, running maxima and sums, output accumulators per map; the
//                               value tile is read once from memory for both), so the difference, the norm over
//                               the head and the scale happen on the accumulators.  Prompt portions and single
//                               tokens of a mixed batch in one launch.
#include "attention_bf16.cuh"

using namespace sprout_attn;

namespace {

constexpr int CHUNK = 128;
constexpr int PARTS = 4;     // value elements per thread in the float32-arithmetic kernel: vdim <= PARTS * CHUNK

// Row of a token: [q: q_vectors * dim | k: kv_heads * maps * dim | v: kv_heads * vdim] (k and v only when `write`; no v
// when `value_from_key`: the value row is then the key row as projected, before rotation and norm, and vdim = maps * dim).
// A warp takes a vector: it rotates the first `rot` elements, then, with `unit_eps` > 0, divides the vector by its root
// mean square over dim (float32; rounded once, on the way out).
constexpr int ROPE_MAX_PER_LANE = 16;        // vectors of up to 512 elements

template <typename T>
__global__ void __launch_bounds__(128)
rope_maps_append_kernel(T* __restrict__ rows, int row_stride, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int table_stride,
                        const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_positions,
                        T* __restrict__ k_cache, T* __restrict__ v_cache, int q_vectors, int kv_heads, int maps, int dim,
                        int rot, int vdim, int page_tokens, int num_pages, int write, float unit_eps, int value_from_key,
                        const float* __restrict__ q_weight, const float* __restrict__ k_weight, float weight_eps,
                        int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int pos = positions[t];
  T* row = rows + (size_t)t * row_stride;
  const int half = rot / 2;
  const bool turn = rot > 0 && pos >= 0 && pos < max_positions;
  if (rot > 0 && !turn && threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_POSITION);
  const float* cs = cos_table + (size_t)(turn ? pos : 0) * half;
  const float* sn = sin_table + (size_t)(turn ? pos : 0) * half;
  int page = -1;
  if (write) {
    page = pos >= 0 ? block_table[(size_t)seq_of_token[t] * table_stride + pos / page_tokens] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
      page = -1;
    }
  }
  const int kw = maps * dim;
  const int vectors = q_vectors + (write ? kv_heads * maps : 0);
  for (int vec = warp; vec < vectors; vec += warps) {
    const bool is_key = vec >= q_vectors;
    if (is_key && page < 0) continue;
    const float* weight = is_key ? k_weight : q_weight;           // the norm before the rotation, when the vector has one
    if (!is_key && !turn && unit_eps <= 0.f && weight == nullptr) continue;   // nothing to do to this query vector
    T* src = row + (size_t)vec * dim;                             // the key vectors follow the query vectors
    float vals[ROPE_MAX_PER_LANE], raw[ROPE_MAX_PER_LANE];
    float before = 1.0f;
    if (weight != nullptr) {
      float sq = 0.f;
#pragma unroll
      for (int j = 0; j < ROPE_MAX_PER_LANE; j++)
        if (lane + 32 * j < dim) {
          const float x = to_float(src[lane + 32 * j]);
          sq = fmaf(x, x, sq);
        }
      before = 1.0f / sqrtf(warp_sum(sq) / (float)dim + weight_eps);
    }
    float squares = 0.f;
#pragma unroll
    for (int j = 0; j < ROPE_MAX_PER_LANE; j++) {
      const int d = lane + 32 * j;
      vals[j] = raw[j] = 0.f;
      if (d < dim) {
        float x = to_float(src[d]);
        raw[j] = x;
        if (weight != nullptr) x = x * before * weight[d];
        if (turn && d < rot) {
          const int i = d < half ? d : d - half, partner = d < half ? d + half : d - half;
          float other = to_float(src[partner]);
          if (weight != nullptr) other = other * before * weight[partner];
          x = d < half ? x * cs[i] - other * sn[i] : x * cs[i] + other * sn[i];
        }
        vals[j] = x;
        squares = fmaf(x, x, squares);
      }
    }
    float factor = 1.0f;
    if (unit_eps > 0.f) factor = 1.0f / sqrtf(warp_sum(squares) / (float)dim + unit_eps);
    __syncwarp();                                                 // every partner element was read before any is rewritten
    if (!is_key) {
#pragma unroll
      for (int j = 0; j < ROPE_MAX_PER_LANE; j++)
        if (lane + 32 * j < dim) src[lane + 32 * j] = from_float<T>(vals[j] * factor);
      continue;
    }
    const int g = (vec - q_vectors) / maps, m = (vec - q_vectors) % maps;
    const size_t at = ((size_t)page * kv_heads + g) * page_tokens + pos % page_tokens;
#pragma unroll
    for (int j = 0; j < ROPE_MAX_PER_LANE; j++) {
      const int d = lane + 32 * j;
      if (d < dim) {
        k_cache[at * kw + m * dim + d] = from_float<T>(vals[j] * factor);
        if (value_from_key) v_cache[at * vdim + m * dim + d] = from_float<T>(raw[j]);
      }
    }
  }
  if (!write || page < 0 || value_from_key) return;
  const T* vrow = row + (size_t)q_vectors * dim + (size_t)kv_heads * kw;
  for (int i = threadIdx.x; i < kv_heads * vdim; i += blockDim.x) {
    const int g = i / vdim, e = i % vdim;
    v_cache[(((size_t)page * kv_heads + g) * page_tokens + pos % page_tokens) * vdim + e] = vrow[i];
  }
}

// The first position that a query at `pos` sees: 0 (causal), pos - size + 1 (a window of `size` positions, itself
// included) or the start of its chunk of `size` positions counted from position 0.
// `keep` (a window only): the first `keep` positions stay visible to every later query, at their own positions.
enum MaskKind : int { MASK_CAUSAL = 0, MASK_WINDOW = 1, MASK_CHUNK = 2 };
// cap * tanh(s / cap) for the bfloat16 kernel: through one exponential, absolute error about cap * 2e-7
__device__ __forceinline__ float soft_cap_fast(float s, float cap, float inv_cap) {
  const float e = __expf(2.0f * s * inv_cap);
  return cap * (1.0f - __fdividef(2.0f, e + 1.0f));
}
__device__ __forceinline__ int first_visible(int kind, int size, int pos) {
  if (kind == MASK_WINDOW) return max(0, pos - size + 1);
  if (kind == MASK_CHUNK) return pos < 0 ? 0 : (pos / size) * size;
  return 0;
}

template <typename T, int MAPS>
__global__ void __launch_bounds__(CHUNK)
multimap_attention_simple_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                                 const T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                                 const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                                 T* __restrict__ out, int out_stride, int heads, int kv_heads, int dim, int vdim,
                                 int page_tokens, int num_pages, float scale, float lambda, float norm_eps,
                                 float out_scale, int mask_kind, int mask_size, int mask_keep, float softcap,
                                 const float* __restrict__ sink, const T* __restrict__ gate, int gate_stride, int* status) {
  extern __shared__ float smem[];
  float* qs = smem;                                   // MAPS * dim
  float* probs = qs + MAPS * dim;                     // MAPS * CHUNK
  float* scratch = probs + MAPS * CHUNK;              // 34
  long long* row_index = (long long*)(scratch + 34 + ((MAPS * dim) & 1));   // CHUNK, 8-byte aligned

  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int g = h / (heads / kv_heads);
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  const int kw = MAPS * dim;
  for (int d = tid; d < kw; d += CHUNK) qs[d] = to_float(q[(size_t)t * q_stride + (size_t)h * kw + d]);
  __syncthreads();

  float m_run[MAPS], l_run[MAPS], acc[MAPS][PARTS];
#pragma unroll
  for (int m = 0; m < MAPS; m++) {
    m_run[m] = -INFINITY;
    l_run[m] = 0.f;
#pragma unroll
    for (int part = 0; part < PARTS; part++) acc[m][part] = 0.f;
  }
  const int lo = first_visible(mask_kind, mask_size, pos);
  const int keep = min(mask_keep, lo);                // kept first positions that the window itself does not reach
  for (int base = 0; base <= pos; base += CHUNK) {
    if (base >= keep && base + CHUNK <= lo) continue; // a chunk of which the query sees nothing
    const int p = base + tid;
    bool valid = (p >= lo || p < keep) && p <= pos;
    long long index = -1;
    if (valid) {
      const int page = table[p / page_tokens];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, SPROUT_STATUS_BAD_PAGE);
        valid = false;
      } else {
        index = ((long long)page * kv_heads + g) * page_tokens + (p % page_tokens);
      }
    }
    float s[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      s[m] = -INFINITY;
      if (valid) {
        const T* key = k_cache + index * kw + m * dim;
        float dot = 0.f;
        for (int d = 0; d < dim; d++) dot = fmaf(qs[m * dim + d], to_float(key[d]), dot);
        s[m] = dot * scale;
        if (softcap > 0.f) s[m] = softcap * tanhf(s[m] / softcap);
      }
    }
    row_index[tid] = index;
    float alpha[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      const float m_new = fmaxf(m_run[m], block_max(s[m], scratch));
      const float e = valid ? expf(s[m] - m_new) : 0.f;
      probs[m * CHUNK + tid] = e;
      const float c_sum = block_sum(e, scratch);
      alpha[m] = (m_run[m] == -INFINITY) ? 0.f : expf(m_run[m] - m_new);
      l_run[m] = l_run[m] * alpha[m] + c_sum;
      m_run[m] = m_new;
    }
    __syncthreads();
    const int count = min(CHUNK, pos - base + 1);
#pragma unroll
    for (int part = 0; part < PARTS; part++) {
      const int e = tid + part * CHUNK;
      if (e < vdim) {
#pragma unroll
        for (int m = 0; m < MAPS; m++) acc[m][part] *= alpha[m];
        for (int j = 0; j < count; j++) {
          const long long r = row_index[j];
          if (r < 0) continue;
          const float v = to_float(v_cache[r * vdim + e]);
#pragma unroll
          for (int m = 0; m < MAPS; m++) acc[m][part] = fmaf(probs[m * CHUNK + j], v, acc[m][part]);
        }
      }
    }
    __syncthreads();
  }
  if (sink != nullptr) {
    // one more term in every map's denominator: exp(sink_h), with no key and no value
    const float extra = sink[h];
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      const float top = fmaxf(m_run[m], extra);
      const float keep = (m_run[m] == -INFINITY) ? 0.f : expf(m_run[m] - top);
      l_run[m] = l_run[m] * keep + expf(extra - top);
#pragma unroll
      for (int part = 0; part < PARTS; part++) acc[m][part] *= keep;
    }
  }
  float o[PARTS];
  float squares = 0.f;
#pragma unroll
  for (int part = 0; part < PARTS; part++) {
    o[part] = acc[0][part] / l_run[0];
    if (MAPS == 2) o[part] -= lambda * (acc[MAPS - 1][part] / l_run[MAPS - 1]);
    if (tid + part * CHUNK < vdim) squares = fmaf(o[part], o[part], squares);
  }
  float factor = out_scale;
  if (norm_eps > 0.f) factor *= 1.0f / sqrtf(block_sum(squares, scratch) / (float)vdim + norm_eps);
  if (gate != nullptr) factor *= 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + h])));
  T* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
#pragma unroll
  for (int part = 0; part < PARTS; part++)
    if (tid + part * CHUNK < vdim) dst[tid + part * CHUNK] = from_float<T>(o[part] * factor);
}


// ------------------------------------------------------------------------------------------ tensor cores
constexpr int MM_ROWS = 64, MM_KEYS = 64, MM_THREADS = 128;

struct MultiMapParams {
  const __nv_bfloat16* q; int q_stride;
  const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;
  const int* block_table; int table_stride;
  const int* q_start; const int* positions;
  __nv_bfloat16* out; int out_stride;
  int requests, heads, kv_heads, page_tokens, num_pages;
  float scale, lambda, norm_eps, out_scale;
  int* status;
  // single-token steps may divide a request's tiles among `ksplit` CTAs (blockIdx.z); each then leaves its maxima, sums
  // and unnormalised accumulators in `partial` [requests, kv_heads, ksplit, 16 rows, maps, 2 + vdim] for the merge kernel
  int ksplit; float* partial;
  // what a query sees (MaskKind and its size), an optional term exp(sink[head]) in every softmax denominator, and an
  // optional gate: the head's output times sigmoid(gate[token * gate_stride + head])
  int mask_kind, mask_size; const float* sink; const __nv_bfloat16* gate; int gate_stride;
  // a window's kept first positions, and the cap on the scaled scores (0: none)
  int mask_keep; float softcap;
};

// What the running maxima are multiplied by on their way into the exponentials: capped scores are already scaled.
__device__ __forceinline__ float score_scale(const MultiMapParams& p) { return p.softcap > 0.f ? 1.0f : p.scale; }

template <int DIM, int VDIM, int MAPS, bool SPLIT>
__global__ void __launch_bounds__(MM_THREADS)
multimap_attention_mma_kernel(const MultiMapParams p) {
  constexpr int KW = MAPS * DIM, KSTRIDE = KW + 8, VSTRIDE = VDIM + 8, KCHUNKS = KW / 8, VCHUNKS = VDIM / 8;
  extern __shared__ __align__(16) unsigned char mm_smem[];
  __nv_bfloat16* sQ = (__nv_bfloat16*)mm_smem;                   // MM_ROWS x KSTRIDE
  __nv_bfloat16* sK = sQ + MM_ROWS * KSTRIDE;                    // 2 x MM_KEYS x KSTRIDE
  __nv_bfloat16* sV = sK + 2 * MM_KEYS * KSTRIDE;                // 2 x MM_KEYS x VSTRIDE
  __shared__ int s_token[MM_ROWS], s_head[MM_ROWS], s_limit[MM_ROWS], s_lo[MM_ROWS];
  __shared__ long long s_row[2][MM_KEYS];

  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.y, group = p.heads / p.kv_heads;
  int tile = blockIdx.x, r = 0;
  for (; r < p.requests; r++) {
    const int tiles = ((p.q_start[r + 1] - p.q_start[r]) * group + MM_ROWS - 1) / MM_ROWS;
    if (tile < tiles) {
      tile = (tile & 1) ? tiles - 1 - (tile >> 1) : (tile >> 1);     // long and short causal tiles in turn
      break;
    }
    tile -= tiles;
  }
  if (r >= p.requests) return;
  const int q0 = p.q_start[r], rows_total = (p.q_start[r + 1] - q0) * group, row_base = tile * MM_ROWS;
  const int* table = p.block_table + (size_t)r * p.table_stride;
  if (tid < MM_ROWS) {
    const int gi = row_base + tid;
    if (gi < rows_total) {
      const int tok = q0 + gi / group;
      s_token[tid] = tok;
      s_head[tid] = g * group + gi % group;
      s_limit[tid] = p.positions[tok];
      s_lo[tid] = first_visible(p.mask_kind, p.mask_size, s_limit[tid]);
    } else {
      s_token[tid] = -1; s_head[tid] = 0; s_limit[tid] = -1; s_lo[tid] = 0;
    }
  }
  __syncthreads();
  const int last_row = min(rows_total, row_base + MM_ROWS) - 1 - row_base;
  const int max_limit = s_limit[last_row];                          // positions grow with the row index
  const int kv_tiles = max_limit / MM_KEYS + 1;
  const int min_lo = s_lo[0];                                       // the first key any row sees: lo grows with the position
  const int tile_lo = min_lo / MM_KEYS;
  // the CTA's tiles: those of the kept first positions that lie before the window's, then the window's up to the last query
  const int keep_tiles = min((p.mask_keep + MM_KEYS - 1) / MM_KEYS, tile_lo);
  const int list_tiles = keep_tiles + (kv_tiles - tile_lo);
  auto tile_of = [&](int i) { return i < keep_tiles ? i : tile_lo + (i - keep_tiles); };

  for (int idx = tid; idx < MM_ROWS * KCHUNKS; idx += MM_THREADS) {
    const int row = idx / KCHUNKS, c = idx % KCHUNKS;
    __nv_bfloat16* dst = sQ + row * KSTRIDE + c * 8;
    if (s_token[row] >= 0) cp_async16(dst, p.q + (size_t)s_token[row] * p.q_stride + (size_t)s_head[row] * KW + c * 8);
    else *(uint4*)dst = make_uint4(0, 0, 0, 0);
  }
  auto find_rows = [&](int t, int buf) {
    if (tid < MM_KEYS) {
      const int key = t * MM_KEYS + tid;
      long long row = -1;
      if ((key >= min_lo || key < p.mask_keep) && key <= max_limit) {
        const int page = table[key / p.page_tokens];
        if (page < 0 || page >= p.num_pages) atomicOr(p.status, SPROUT_STATUS_BAD_PAGE);
        else row = ((long long)page * p.kv_heads + g) * p.page_tokens + key % p.page_tokens;
      }
      s_row[buf][tid] = row;
    }
  };
  auto load_tile = [&](int buf) {
    for (int idx = tid; idx < MM_KEYS * KCHUNKS; idx += MM_THREADS) {
      const int row = idx / KCHUNKS, c = idx % KCHUNKS;
      const long long at = s_row[buf][row];
      __nv_bfloat16* dst = sK + (buf * MM_KEYS + row) * KSTRIDE + c * 8;
      if (at >= 0) cp_async16(dst, p.k_cache + at * KW + c * 8);
      else *(uint4*)dst = make_uint4(0, 0, 0, 0);
    }
    for (int idx = tid; idx < MM_KEYS * VCHUNKS; idx += MM_THREADS) {
      const int row = idx / VCHUNKS, c = idx % VCHUNKS;
      const long long at = s_row[buf][row];
      __nv_bfloat16* dst = sV + (buf * MM_KEYS + row) * VSTRIDE + c * 8;
      if (at >= 0) cp_async16(dst, p.v_cache + at * VDIM + c * 8);
      else *(uint4*)dst = make_uint4(0, 0, 0, 0);
    }
  };
  const int first_tile = SPLIT ? (int)blockIdx.z : 0, tile_step = SPLIT ? p.ksplit : 1;    // this CTA's tiles: every tile_step-th of the list
  if (first_tile < list_tiles) find_rows(tile_of(first_tile), 0);
  __syncthreads();
  if (first_tile < list_tiles) load_tile(0);
  cp_async_commit();

  // SPLIT (a step in which no request has more than 16 rows: single tokens, the heads of one key/value group): a CTA
  // divides every tile's keys among its warps instead of its rows, and the warps' partial results are merged at the end.
  constexpr bool split = SPLIT;
  const int qrow = split ? 0 : warp * 16;             // the warp's 16 rows
  constexpr int nk = split ? 1 : MM_KEYS / 16;        // blocks of 16 keys of a tile that the warp takes, from key kb on
  const int kb = split ? warp * 16 : 0;
  const int gr = lane >> 2, qc = lane & 3;
  const int my_row0 = qrow + gr, my_row1 = my_row0 + 8;
  const int limit0 = s_limit[my_row0], limit1 = s_limit[my_row1];
  const int lo0 = s_lo[my_row0], lo1 = s_lo[my_row1];
  float m0[MAPS], m1[MAPS], l0[MAPS], l1[MAPS];
  float o[MAPS][VDIM / 8][4];
#pragma unroll
  for (int m = 0; m < MAPS; m++) {
    m0[m] = m1[m] = -INFINITY;
    l0[m] = l1[m] = 0.f;
#pragma unroll
    for (int i = 0; i < VDIM / 8; i++) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.f;
  }
  const float scale_log2 = score_scale(p) * 1.4426950408889634f;
  const float inv_cap = p.softcap > 0.f ? 1.0f / p.softcap : 0.f;
  const int warp_min_limit = s_limit[min(qrow, last_row)];
  const int warp_min_lo = s_lo[min(qrow, last_row)], warp_max_lo = s_lo[min(qrow + 15, last_row)];

  int buf = 1;
  for (int ti = first_tile; ti < list_tiles; ti += tile_step) {
    const int t = tile_of(ti);
    buf ^= 1;
    if (ti + tile_step < list_tiles) find_rows(tile_of(ti + tile_step), buf ^ 1);
    __syncthreads();                                   // rows visible; everyone is done with buffer buf ^ 1
    if (ti + tile_step < list_tiles) load_tile(buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();                                // tile t (and Q) have landed
    __syncthreads();
    const __nv_bfloat16* tK = sK + buf * MM_KEYS * KSTRIDE;
    const __nv_bfloat16* tV = sV + buf * MM_KEYS * VSTRIDE;
    const int kv0 = t * MM_KEYS;
    if (kv0 + kb > s_limit[min(qrow + 15, last_row)] || (kv0 + kb + nk * 16 <= warp_min_lo && kv0 + kb >= p.mask_keep)) continue;   // no row of this warp sees its keys of the tile
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      float s[MM_KEYS / 8][4];
#pragma unroll
      for (int i = 0; i < MM_KEYS / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DIM / 16; kk++) {
        uint32_t a[4];
        ldmatrix_x4(a, sQ + (qrow + (lane & 7) + ((lane >> 3) & 1) * 8) * KSTRIDE + m * DIM + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n2 = 0; n2 < MM_KEYS / 16; n2++) {
          if (n2 >= nk) break;
          uint32_t b[4];
          ldmatrix_x4(b, tK + (kb + n2 * 16 + (lane & 7) + (lane >> 4) * 8) * KSTRIDE + m * DIM + kk * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * n2], a, b[0], b[1]);
          mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
        }
      }
      if (p.softcap > 0.f) {
        const float cap = p.softcap, pre = p.scale;
#pragma unroll
        for (int i = 0; i < MM_KEYS / 8; i++) {
          if (i >= 2 * nk) break;
#pragma unroll
          for (int c = 0; c < 4; c++) s[i][c] = soft_cap_fast(s[i][c] * pre, cap, inv_cap);
        }
      }
      float t_max0 = -INFINITY, t_max1 = -INFINITY;
      if (kv0 + kb + nk * 16 - 1 > warp_min_limit) {
#pragma unroll
        for (int i = 0; i < MM_KEYS / 8; i++) {
          if (i >= 2 * nk) break;
          const int key = kv0 + kb + i * 8 + qc * 2;
          if (key > limit0) s[i][0] = -INFINITY;
          if (key + 1 > limit0) s[i][1] = -INFINITY;
          if (key > limit1) s[i][2] = -INFINITY;
          if (key + 1 > limit1) s[i][3] = -INFINITY;
        }
      }
      if (kv0 + kb < warp_max_lo) {                                  // keys before a row's window or chunk
#pragma unroll
        for (int i = 0; i < MM_KEYS / 8; i++) {
          if (i >= 2 * nk) break;
          const int key = kv0 + kb + i * 8 + qc * 2;
          const int kept = p.mask_keep;
          if (key < lo0 && key >= kept) s[i][0] = -INFINITY;
          if (key + 1 < lo0 && key + 1 >= kept) s[i][1] = -INFINITY;
          if (key < lo1 && key >= kept) s[i][2] = -INFINITY;
          if (key + 1 < lo1 && key + 1 >= kept) s[i][3] = -INFINITY;
        }
      }
#pragma unroll
      for (int i = 0; i < MM_KEYS / 8; i++) {
        if (i >= 2 * nk) break;
        t_max0 = fmaxf(t_max0, fmaxf(s[i][0], s[i][1]));
        t_max1 = fmaxf(t_max1, fmaxf(s[i][2], s[i][3]));
      }
      t_max0 = fmaxf(t_max0, __shfl_xor_sync(0xffffffffu, t_max0, 1));
      t_max0 = fmaxf(t_max0, __shfl_xor_sync(0xffffffffu, t_max0, 2));
      t_max1 = fmaxf(t_max1, __shfl_xor_sync(0xffffffffu, t_max1, 1));
      t_max1 = fmaxf(t_max1, __shfl_xor_sync(0xffffffffu, t_max1, 2));
      const float n0 = fmaxf(m0[m], t_max0), n1 = fmaxf(m1[m], t_max1);     // running maxima of the unscaled scores
      const float base0 = n0 == -INFINITY ? 0.f : n0 * scale_log2, base1 = n1 == -INFINITY ? 0.f : n1 * scale_log2;
      const float alpha0 = m0[m] == -INFINITY ? 0.f : exp2f(m0[m] * scale_log2 - base0);
      const float alpha1 = m1[m] == -INFINITY ? 0.f : exp2f(m1[m] * scale_log2 - base1);
      m0[m] = n0; m1[m] = n1;
      l0[m] *= alpha0; l1[m] *= alpha1;
#pragma unroll
      for (int i = 0; i < VDIM / 8; i++) { o[m][i][0] *= alpha0; o[m][i][1] *= alpha0; o[m][i][2] *= alpha1; o[m][i][3] *= alpha1; }
#pragma unroll
      for (int i = 0; i < MM_KEYS / 8; i++) {
        if (i >= 2 * nk) break;
        s[i][0] = exp2f(fmaf(s[i][0], scale_log2, -base0)); s[i][1] = exp2f(fmaf(s[i][1], scale_log2, -base0));
        s[i][2] = exp2f(fmaf(s[i][2], scale_log2, -base1)); s[i][3] = exp2f(fmaf(s[i][3], scale_log2, -base1));
        l0[m] += s[i][0] + s[i][1];
        l1[m] += s[i][2] + s[i][3];
      }
#pragma unroll
      for (int kk = 0; kk < MM_KEYS / 16; kk++) {
        if (kk >= nk) break;
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d2 = 0; d2 < VDIM / 16; d2++) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, tV + (kb + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VSTRIDE + d2 * 16 + (lane >> 4) * 8);
          mma_bf16(o[m][2 * d2], a, b[0], b[1]);
          mma_bf16(o[m][2 * d2 + 1], a, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

  // per row: a_0 - lambda a_1, the norm over the head's values (the quad holds a row), the scale
  float inv0[MAPS], inv1[MAPS];
#pragma unroll
  for (int m = 0; m < MAPS; m++) {
    l0[m] += __shfl_xor_sync(0xffffffffu, l0[m], 1); l0[m] += __shfl_xor_sync(0xffffffffu, l0[m], 2);
    l1[m] += __shfl_xor_sync(0xffffffffu, l1[m], 1); l1[m] += __shfl_xor_sync(0xffffffffu, l1[m], 2);
  }
  if (split) {
    // the warps hold the same rows over different keys: warp 0 merges them, in the warps' order
    constexpr int PER = MAPS * (VDIM / 8 * 4 + 4);
    float* slots = (float*)mm_smem;
    __syncthreads();                                   // the tiles are no longer read
    float* mine = slots + (size_t)(warp * 32 + lane) * PER;
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      float* at = mine + m * (VDIM / 8 * 4 + 4);
      at[0] = m0[m]; at[1] = m1[m]; at[2] = l0[m]; at[3] = l1[m];
#pragma unroll
      for (int i = 0; i < VDIM / 8; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) at[4 + i * 4 + c] = o[m][i][c];
    }
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      float top0 = -INFINITY, top1 = -INFINITY;
      for (int w = 0; w < MM_THREADS / 32; w++) {
        const float* at = slots + (size_t)(w * 32 + lane) * PER + m * (VDIM / 8 * 4 + 4);
        top0 = fmaxf(top0, at[0]);
        top1 = fmaxf(top1, at[1]);
      }
      l0[m] = l1[m] = 0.f;
      m0[m] = top0;
      m1[m] = top1;
#pragma unroll
      for (int i = 0; i < VDIM / 8; i++) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.f;
      for (int w = 0; w < MM_THREADS / 32; w++) {
        const float* at = slots + (size_t)(w * 32 + lane) * PER + m * (VDIM / 8 * 4 + 4);
        const float f0 = at[0] == -INFINITY ? 0.f : exp2f((at[0] - top0) * scale_log2);
        const float f1 = at[1] == -INFINITY ? 0.f : exp2f((at[1] - top1) * scale_log2);
        l0[m] = fmaf(at[2], f0, l0[m]);
        l1[m] = fmaf(at[3], f1, l1[m]);
#pragma unroll
        for (int i = 0; i < VDIM / 8; i++) {
          o[m][i][0] = fmaf(at[4 + i * 4], f0, o[m][i][0]);
          o[m][i][1] = fmaf(at[4 + i * 4 + 1], f0, o[m][i][1]);
          o[m][i][2] = fmaf(at[4 + i * 4 + 2], f1, o[m][i][2]);
          o[m][i][3] = fmaf(at[4 + i * 4 + 3], f1, o[m][i][3]);
        }
      }
    }
  }
  if (SPLIT && p.ksplit > 1) {
    // this CTA saw a share of the keys: what it has goes to the merge kernel
    float* base = p.partial + ((((size_t)r * p.kv_heads + g) * p.ksplit + blockIdx.z) * 16) * MAPS * (2 + VDIM);
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      float* row0 = base + ((size_t)my_row0 * MAPS + m) * (2 + VDIM);
      float* row1 = base + ((size_t)my_row1 * MAPS + m) * (2 + VDIM);
      if (qc == 0) { row0[0] = m0[m]; row0[1] = l0[m]; row1[0] = m1[m]; row1[1] = l1[m]; }
#pragma unroll
      for (int i = 0; i < VDIM / 8; i++) {
        *(float2*)(row0 + 2 + i * 8 + qc * 2) = make_float2(o[m][i][0], o[m][i][1]);
        *(float2*)(row1 + 2 + i * 8 + qc * 2) = make_float2(o[m][i][2], o[m][i][3]);
      }
    }
    return;
  }
  if (p.sink != nullptr) {
    // exp(sink) joins every map's denominator: rescale to the larger of the running maximum and the sink
    const float sk0 = p.sink[s_head[my_row0]] * 1.4426950408889634f, sk1 = p.sink[s_head[my_row1]] * 1.4426950408889634f;
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      const float b0 = m0[m] == -INFINITY ? -INFINITY : m0[m] * scale_log2, b1 = m1[m] == -INFINITY ? -INFINITY : m1[m] * scale_log2;
      const float t0 = fmaxf(b0, sk0), t1 = fmaxf(b1, sk1);
      const float k0 = b0 == -INFINITY ? 0.f : exp2f(b0 - t0), k1 = b1 == -INFINITY ? 0.f : exp2f(b1 - t1);
      l0[m] = l0[m] * k0 + exp2f(sk0 - t0);
      l1[m] = l1[m] * k1 + exp2f(sk1 - t1);
#pragma unroll
      for (int i = 0; i < VDIM / 8; i++) { o[m][i][0] *= k0; o[m][i][1] *= k0; o[m][i][2] *= k1; o[m][i][3] *= k1; }
    }
  }
#pragma unroll
  for (int m = 0; m < MAPS; m++) {
    inv0[m] = 1.0f / l0[m];
    inv1[m] = 1.0f / l1[m];
  }
  float sq0 = 0.f, sq1 = 0.f;
#pragma unroll
  for (int i = 0; i < VDIM / 8; i++) {
#pragma unroll
    for (int c = 0; c < 2; c++) {
      float v0 = o[0][i][c] * inv0[0], v1 = o[0][i][2 + c] * inv1[0];
      if (MAPS == 2) {
        v0 -= p.lambda * (o[MAPS - 1][i][c] * inv0[MAPS - 1]);
        v1 -= p.lambda * (o[MAPS - 1][i][2 + c] * inv1[MAPS - 1]);
      }
      o[0][i][c] = v0;
      o[0][i][2 + c] = v1;
      sq0 = fmaf(v0, v0, sq0);
      sq1 = fmaf(v1, v1, sq1);
    }
  }
  float f0 = p.out_scale, f1 = p.out_scale;
  if (p.norm_eps > 0.f) {
    sq0 += __shfl_xor_sync(0xffffffffu, sq0, 1); sq0 += __shfl_xor_sync(0xffffffffu, sq0, 2);
    sq1 += __shfl_xor_sync(0xffffffffu, sq1, 1); sq1 += __shfl_xor_sync(0xffffffffu, sq1, 2);
    f0 *= 1.0f / sqrtf(sq0 / (float)VDIM + p.norm_eps);
    f1 *= 1.0f / sqrtf(sq1 / (float)VDIM + p.norm_eps);
  }
  if (p.gate != nullptr) {
    if (s_token[my_row0] >= 0) f0 *= 1.0f / (1.0f + expf(-__bfloat162float(p.gate[(size_t)s_token[my_row0] * p.gate_stride + s_head[my_row0]])));
    if (s_token[my_row1] >= 0) f1 *= 1.0f / (1.0f + expf(-__bfloat162float(p.gate[(size_t)s_token[my_row1] * p.gate_stride + s_head[my_row1]])));
  }
  if (s_token[my_row0] >= 0) {
    __nv_bfloat16* dst = p.out + (size_t)s_token[my_row0] * p.out_stride + (size_t)s_head[my_row0] * VDIM + qc * 2;
#pragma unroll
    for (int i = 0; i < VDIM / 8; i++) *(__nv_bfloat162*)(dst + i * 8) = __floats2bfloat162_rn(o[0][i][0] * f0, o[0][i][1] * f0);
  }
  if (s_token[my_row1] >= 0) {
    __nv_bfloat16* dst = p.out + (size_t)s_token[my_row1] * p.out_stride + (size_t)s_head[my_row1] * VDIM + qc * 2;
#pragma unroll
    for (int i = 0; i < VDIM / 8; i++) *(__nv_bfloat162*)(dst + i * 8) = __floats2bfloat162_rn(o[0][i][2] * f1, o[0][i][3] * f1);
  }
}

// One block per (request, key/value head, row): the CTAs' shares of a request's keys into the head's output.
template <int MAPS>
__global__ void __launch_bounds__(128)
multimap_merge_kernel(const MultiMapParams p, int vdim) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, g = blockIdx.y, row = blockIdx.z, group = p.heads / p.kv_heads;
  const int q0 = p.q_start[r], rows_total = (p.q_start[r + 1] - q0) * group;
  if (row >= rows_total) return;
  const int token = q0 + row / group, head = g * group + row % group;
  const float scale_log2 = score_scale(p) * 1.4426950408889634f;
  const float* base = p.partial + (((size_t)r * p.kv_heads + g) * p.ksplit * 16 + row) * MAPS * (2 + vdim);
  const size_t share = (size_t)16 * MAPS * (2 + vdim);
  float v[2] = {0.f, 0.f};                             // columns threadIdx.x and threadIdx.x + 128
#pragma unroll
  for (int m = 0; m < MAPS; m++) {
    float top = -INFINITY;
    for (int z = 0; z < p.ksplit; z++) top = fmaxf(top, base[z * share + m * (2 + vdim)]);
    float sum = 0.f, a[2] = {0.f, 0.f};
    float top_log2 = top == -INFINITY ? -INFINITY : top * scale_log2;     // the shares' maxima are those of the unscaled scores
    if (p.sink != nullptr) {
      const float sk = p.sink[head] * 1.4426950408889634f;
      top_log2 = fmaxf(top_log2, sk);
      sum = exp2f(sk - top_log2);
    }
    for (int z = 0; z < p.ksplit; z++) {
      const float* at = base + z * share + m * (2 + vdim);
      const float f = at[0] == -INFINITY ? 0.f : exp2f(at[0] * scale_log2 - top_log2);
      sum = fmaf(at[1], f, sum);
#pragma unroll
      for (int part = 0; part < 2; part++)
        if (threadIdx.x + part * 128 < vdim) a[part] = fmaf(at[2 + threadIdx.x + part * 128], f, a[part]);
    }
#pragma unroll
    for (int part = 0; part < 2; part++) v[part] += (m == 0 ? 1.0f : -p.lambda) * (a[part] / sum);
  }
  float squares = 0.f;
#pragma unroll
  for (int part = 0; part < 2; part++)
    if (threadIdx.x + part * 128 < vdim) squares = fmaf(v[part], v[part], squares);
  float factor = p.out_scale;
  if (p.norm_eps > 0.f) factor *= 1.0f / sqrtf(block_sum(squares, scratch) / (float)vdim + p.norm_eps);
  if (p.gate != nullptr) factor *= 1.0f / (1.0f + expf(-__bfloat162float(p.gate[(size_t)token * p.gate_stride + head])));
  __nv_bfloat16* dst = p.out + (size_t)token * p.out_stride + (size_t)head * vdim;
#pragma unroll
  for (int part = 0; part < 2; part++)
    if (threadIdx.x + part * 128 < vdim) dst[threadIdx.x + part * 128] = __float2bfloat16_rn(v[part] * factor);
}

template <int DIM, int VDIM, int MAPS, bool SPLIT>
int launch_multimap(const MultiMapParams& p, int grid_x, cudaStream_t stream) {
  const int tiles_bytes = (3 * MM_ROWS * (MAPS * DIM + 8) + 2 * MM_KEYS * (VDIM + 8)) * 2;
  const int merge_bytes = MM_THREADS * MAPS * (VDIM / 8 * 4 + 4) * 4;         // the warps' partial results of a 16-row CTA
  const int smem = tiles_bytes > merge_bytes ? tiles_bytes : merge_bytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(multimap_attention_mma_kernel<DIM, VDIM, MAPS, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return sprout_fail("multimap_attention_mma: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(err));
    configured = true;
  }
  sprout_launch(multimap_attention_mma_kernel<DIM, VDIM, MAPS, SPLIT>, dim3(grid_x, p.kv_heads, SPLIT ? p.ksplit : 1), dim3(MM_THREADS),
                smem, stream, p);
  if (int code = sprout_check_launch("multimap_attention_mma")) return code;
  if (SPLIT && p.ksplit > 1) {
    sprout_launch(multimap_merge_kernel<MAPS>, dim3(p.requests, p.kv_heads, 16), dim3(128), 0, stream, p, VDIM);
    return sprout_check_launch("multimap_merge");
  }
  return 0;
}

bool mma_sizes(int maps, int dim, int vdim) {
  return (maps == 1 || maps == 2) && ((dim == 32 && vdim == 64) || (dim == 64 && vdim == 64) || (dim == 64 && vdim == 128) ||
                                      (dim == 128 && vdim == 128) || (dim == 16 && vdim == 32) || (dim == 32 && vdim == 32));
}

}  // namespace

SPROUT_API int sprout_multimap_attention_mma_supported(int maps, int dim, int vdim) { return mma_sizes(maps, dim, vdim) ? 1 : 0; }

// Floats of scratch that a step of single tokens needs when a request's keys are divided among `ksplit` CTAs.
SPROUT_API long long sprout_multimap_partial_floats(int requests, int kv_heads, int maps, int vdim, int ksplit) {
  return (long long)requests * kv_heads * ksplit * 16 * maps * (2 + vdim);
}

// bfloat16 only.  `tiles` bounds the (request, 64 rows) tiles of the batch: sum over requests of
// ceil(tokens * heads / kv_heads / 64), or any larger number; `max_q_len` is the most tokens any request brings.
SPROUT_API int sprout_multimap_attention_mma(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                             const int* block_table, int table_stride, const int* q_start,
                                             const int* positions, void* out, int out_stride, int requests, int tiles,
                                             int max_q_len, int heads, int kv_heads, int maps, int dim, int vdim, int page_tokens,
                                             int num_pages, float scale, float lambda, float norm_eps, float out_scale,
                                             int ksplit, float* partial, int mask_kind, int mask_size, const float* sink,
                                             const void* gate, int gate_stride, int mask_keep, float softcap, int* status,
                                             cudaStream_t stream) {
  SPROUT_REQUIRE(q && k_cache && v_cache && block_table && q_start && positions && out && status, "multimap_attention_mma: null pointer");
  SPROUT_REQUIRE(requests > 0 && tiles > 0 && max_q_len > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && page_tokens > 0 &&
                 num_pages > 0, "multimap_attention_mma: bad sizes");
  SPROUT_REQUIRE(mma_sizes(maps, dim, vdim), "multimap_attention_mma: no kernel for %d maps of %d with values of %d", maps, dim, vdim);
  SPROUT_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 &&
                 ((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)out & 3) == 0, "multimap_attention_mma: rows must start on 16-byte boundaries");
  SPROUT_REQUIRE(kv_heads <= 65535, "multimap_attention_mma: too many key/value heads");
  MultiMapParams p{(const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
                   table_stride, q_start, positions, (__nv_bfloat16*)out, out_stride, requests, heads, kv_heads, page_tokens,
                   num_pages, scale, lambda, norm_eps, out_scale, status, ksplit, partial, mask_kind, mask_size, sink,
                   (const __nv_bfloat16*)gate, gate_stride, mask_keep, softcap};
  SPROUT_REQUIRE(mask_kind == MASK_CAUSAL || ((mask_kind == MASK_WINDOW || mask_kind == MASK_CHUNK) && mask_size > 0),
                 "multimap_attention_mma: a window or a chunk needs a positive size");
  SPROUT_REQUIRE(mask_keep >= 0 && (mask_keep == 0 || mask_kind == MASK_WINDOW) && softcap >= 0.f,
                 "multimap_attention_mma: only a window keeps first positions; the cap is not negative");
  SPROUT_REQUIRE(!gate || gate_stride >= heads, "multimap_attention_mma: gate rows hold a number per head");
  SPROUT_REQUIRE(ksplit >= 1 && ksplit <= 64 && (ksplit == 1 || (partial && max_q_len * (heads / kv_heads) <= 16)),
                 "multimap_attention_mma: keys are divided among CTAs in single-token steps only, with scratch for the shares");
  const bool split = max_q_len * (heads / kv_heads) <= 16;
#define PICK(D, V)                                                                                              \
  if (dim == D && vdim == V) {                                                                                  \
    if (split) return maps == 2 ? launch_multimap<D, V, 2, true>(p, tiles, stream) : launch_multimap<D, V, 1, true>(p, tiles, stream); \
    return maps == 2 ? launch_multimap<D, V, 2, false>(p, tiles, stream) : launch_multimap<D, V, 1, false>(p, tiles, stream);         \
  }
  PICK(32, 64) PICK(64, 64) PICK(64, 128) PICK(128, 128) PICK(16, 32) PICK(32, 32)
#undef PICK
  return sprout_fail("multimap_attention_mma: no kernel for these sizes");
}

SPROUT_API int sprout_rope_maps_append(void* rows, int row_stride, int dtype, const int* positions, const int* seq_of_token,
                                       const int* block_table, int table_stride, const float* cos_table,
                                       const float* sin_table, int max_positions, void* k_cache, void* v_cache, int tokens,
                                       int q_vectors, int kv_heads, int maps, int dim, int rot, int vdim, int page_tokens,
                                       int num_pages, int write, float unit_eps, int value_from_key, const float* q_weight,
                                       const float* k_weight, float weight_eps, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(rows && positions && status && tokens > 0 && q_vectors > 0 && dim > 0 && maps > 0, "rope_maps_append: bad arguments");
  SPROUT_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dim, "rope_maps_append: the rotated width must be even and at most dim");
  SPROUT_REQUIRE(rot == 0 || (cos_table && sin_table && max_positions > 0), "rope_maps_append: tables are missing");
  SPROUT_REQUIRE(!write || (k_cache && v_cache && seq_of_token && block_table && kv_heads > 0 && vdim > 0 && page_tokens > 0 &&
                            num_pages > 0), "rope_maps_append: the cache is missing");
  SPROUT_REQUIRE(dim <= 32 * ROPE_MAX_PER_LANE, "rope_maps_append: vectors of up to %d elements (got %d)", 32 * ROPE_MAX_PER_LANE, dim);
  SPROUT_REQUIRE(!value_from_key || vdim == maps * dim, "rope_maps_append: values that are the keys have the keys' width");
  SPROUT_REQUIRE((!q_weight && !k_weight) || weight_eps > 0.f, "rope_maps_append: a norm before the rotation needs a positive eps");
  const int need = q_vectors * dim + (write ? kv_heads * (maps * dim + (value_from_key ? 0 : vdim)) : 0);
  SPROUT_REQUIRE(row_stride >= need, "rope_maps_append: rows of %d elements, %d needed", row_stride, need);
  if (dtype == SPROUT_F32)
    sprout_launch(rope_maps_append_kernel<float>, dim3(tokens), dim3(128), 0, stream, (float*)rows, row_stride, positions,
                  seq_of_token, block_table, table_stride, cos_table, sin_table, max_positions, (float*)k_cache,
                  (float*)v_cache, q_vectors, kv_heads, maps, dim, rot, vdim, page_tokens, num_pages, write, unit_eps,
                  value_from_key, q_weight, k_weight, weight_eps, status);
  else if (dtype == SPROUT_BF16)
    sprout_launch(rope_maps_append_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, (__nv_bfloat16*)rows, row_stride,
                  positions, seq_of_token, block_table, table_stride, cos_table, sin_table, max_positions,
                  (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, q_vectors, kv_heads, maps, dim, rot, vdim, page_tokens,
                  num_pages, write, unit_eps, value_from_key, q_weight, k_weight, weight_eps, status);
  else
    return sprout_fail("rope_maps_append: unknown dtype %d", dtype);
  return sprout_check_launch("rope_maps_append");
}

SPROUT_API int sprout_multimap_attention_simple(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                                const int* block_table, int table_stride, const int* seq_of_token,
                                                const int* positions, void* out, int out_stride, int dtype, int tokens,
                                                int heads, int kv_heads, int maps, int dim, int vdim, int page_tokens,
                                                int num_pages, float scale, float lambda, float norm_eps, float out_scale,
                                                int mask_kind, int mask_size, const float* sink, const void* gate,
                                                int gate_stride, int mask_keep, float softcap, int* status,
                                                cudaStream_t stream) {
  SPROUT_REQUIRE(q && k_cache && v_cache && block_table && seq_of_token && positions && out && status, "multimap_attention: null pointer");
  SPROUT_REQUIRE(tokens > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && page_tokens > 0 && num_pages > 0,
                 "multimap_attention: bad sizes");
  SPROUT_REQUIRE(maps == 1 || maps == 2, "multimap_attention: one or two maps per head (got %d)", maps);
  SPROUT_REQUIRE(dim > 0 && vdim > 0 && vdim <= PARTS * CHUNK, "multimap_attention: value rows of up to %d elements (got %d)", PARTS * CHUNK, vdim);
  SPROUT_REQUIRE(heads <= 65535, "multimap_attention: too many heads");
  SPROUT_REQUIRE(mask_kind == MASK_CAUSAL || ((mask_kind == MASK_WINDOW || mask_kind == MASK_CHUNK) && mask_size > 0),
                 "multimap_attention: a window or a chunk needs a positive size");
  SPROUT_REQUIRE(!gate || gate_stride >= heads, "multimap_attention: gate rows hold a number per head");
  SPROUT_REQUIRE(mask_keep >= 0 && (mask_keep == 0 || mask_kind == MASK_WINDOW) && softcap >= 0.f,
                 "multimap_attention: only a window keeps first positions; the cap is not negative");
  const size_t smem = (size_t)(maps * dim + maps * CHUNK + 36) * sizeof(float) + CHUNK * sizeof(long long);
  SPROUT_REQUIRE(smem <= 48 * 1024, "multimap_attention: key vectors too long (%d)", dim);
  dim3 grid(tokens, heads);
#define LAUNCH(T, M)                                                                                                      \
  sprout_launch(multimap_attention_simple_kernel<T, M>, grid, dim3(CHUNK), smem, stream, (const T*)q, q_stride,           \
                (const T*)k_cache, (const T*)v_cache, block_table, table_stride, seq_of_token, positions, (T*)out,        \
                out_stride, heads, kv_heads, dim, vdim, page_tokens, num_pages, scale, lambda, norm_eps, out_scale,    \
                mask_kind, mask_size, mask_keep, softcap, sink, (const T*)gate, gate_stride, status)
  if (dtype == SPROUT_F32) {
    if (maps == 1) LAUNCH(float, 1); else LAUNCH(float, 2);
  } else if (dtype == SPROUT_BF16) {
    if (maps == 1) LAUNCH(__nv_bfloat16, 1); else LAUNCH(__nv_bfloat16, 2);
  } else {
    return sprout_fail("multimap_attention: unknown dtype %d", dtype);
  }
#undef LAUNCH
  return sprout_check_launch("multimap_attention_simple");
}
