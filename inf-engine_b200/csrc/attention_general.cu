// Paged causal attention for any mix of prompt portions and decode tokens, any
// head size up to 256 (keys and values each their own), any number of heads and groups,
// an optional window.  float32 arithmetic on CUDA cores with float32 or
// bfloat16 storage: this is the kernel of the true 32-bit path and the fallback
// of the bfloat16 path for sizes that the tensor-core kernels do not take.
//
// Formula (engine/llama_attention.py:106-137): for query token t of a request at
// absolute position p = ctx_before + t and query head h served by kv head
// c = h / group,  out = softmax(q k^T * scale + mask) v  over the keys j <= p
// (and j > p - window when a window is set).  Keys and values are read from the
// request's pages through its block table; the step's own tokens were written
// there before this kernel runs, so every cut of the work sees the same keys.
// An optional additive term enters the score before the softmax: a float32 table
// bias[head][distance], distance = p - j clamped to the table's last column
// (position encodings that bias scores by how far back a key lies).  An optional
// float32 multiplier per query head scales the score before that term is added
// (a learned temperature of each head), and values may have another head size
// than queries and keys (hd_v; the pools are laid out with their own sizes).  Beside a window the first
// `keep_first` keys of the sequence may stay visible to every later query, at their true positions, and the
// output may take a multiplier (a mixer that is one of several summed side by side).  With `chunk` a query at position
// p sees keys from floor(p / chunk) * chunk on only (chunks are counted from the sequence's start, whatever the cut).
// Several key heads may share one value head (`n_v_heads` less than the key heads: two score maps over the same
// values), and the values may be the first dimensions of the key rows themselves (`v_row`: a compressed key/value
// vector that is stored once).
//
// Work split: a block takes one (request, kv head) and a tile of 32
// (token, head-in-group) pairs, so the `group` query heads that share a kv head
// also share every key tile that is loaded.  Keys are walked in tiles of 32 at
// absolute multiples of 32, in ascending order, with an online softmax; the
// sequence of tiles that a (token, head) sees is the same however the tokens
// were cut into steps.
#include "common.cuh"

#define AG_ROWS 32
#define AG_KEYS 32
#define AG_THREADS 256
#define AG_MAX_ACC 32  // head_dim / 8 accumulators per thread, head_dim <= 256

struct AttnGeneralParams {
  const void* q;
  void* out;
  const void* kpool;
  const void* vpool;
  const int* block_table;
  const int* q_start;
  const int* ctx_before;
  const int* work_req;
  const int* work_pair0;
  int q_stride, out_stride, table_stride;
  int n_work, n_heads, n_kv_heads, hd, page_size, window;
  float scale;
  const float* score_bias;  // [n_heads][bias_dists] or null
  int bias_dists;
  const float* head_scale;  // [n_heads] or null: the score is scale * head_scale[head] * (q . k)
  int hd_v;                 // head size of the values and of the output
  int keep_first;           // beside a window: keys at positions below this stay visible to every later query
  float out_scale;          // multiplier of the output
  int chunk;                // > 0: a query sees only keys of its own chunk of this many positions (counted from position 0)
  int n_v_heads;            // value heads in the value pool; kv head c reads value head c / (n_kv_heads / n_v_heads)
  int v_row;                // elements between two value rows of the value pool (the value size, or a key row's size
                            // when the values are the first dimensions of the keys and both pools are one)
  const float* sink;        // [n_heads] or null: the softmax's denominator also holds exp(sink[head]): a learned
                            // logit beside the keys' scores that `scale` does not multiply and that weighs nothing
};

// the normaliser of a row whose visible keys gave the sum l at the maximum m, with the sink's term added
__device__ __forceinline__ float inv_with_sink(float l, float m, const float* sink, int head, float out_scale) {
  if (sink == nullptr || m == -INFINITY) return l > 0.f ? out_scale / l : 0.f;
  const float sk = sink[head];
  const float m2 = fmaxf(m, sk);
  const float f = expf(m - m2);
  return out_scale * f / (l * f + expf(sk - m2));
}

template <typename T>
__global__ void __launch_bounds__(AG_THREADS) attention_general_kernel(AttnGeneralParams p) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int hd = p.hd, hdv = p.hd_v;
  const int ldq = hd + 1;
  float* Qs = smem;                      // [ROWS][hd+1]
  float* Ks = Qs + AG_ROWS * ldq;        // [KEYS][hd+1]
  float* Vs = Ks + AG_KEYS * ldq;        // [KEYS][hd]
  float* Ps = Vs + AG_KEYS * hdv;        // [ROWS][KEYS+1]  (Vs is [KEYS][hdv])

  const int w = blockIdx.x;
  const int c = blockIdx.y;              // kv head
  const int r_id = p.work_req[w];
  const int pair0 = p.work_pair0[w];
  const int group = p.n_heads / p.n_kv_heads;
  const int q0 = p.q_start[r_id];
  const int q_len = p.q_start[r_id + 1] - q0;
  const int ctx = p.ctx_before[r_id];
  const int n_pairs = q_len * group;
  const int* table = p.block_table + (size_t)r_id * p.table_stride;
  const T* q = (const T*)p.q;
  const T* kpool = (const T*)p.kpool;
  const T* vpool = (const T*)p.vpool;

  const int tid = threadIdx.x;
  const int row = tid >> 3;              // 0..31
  const int sub = tid & 7;               // 0..7

  // stage the tile's queries
  for (int idx = tid; idx < AG_ROWS * hd; idx += AG_THREADS) {
    const int r = idx / hd, d = idx - r * hd;
    const int pr = pair0 + r;
    float val = 0.f;
    if (pr < n_pairs) {
      const int t = pr / group, j = pr - t * group;
      val = to_f32(q[(size_t)(q0 + t) * p.q_stride + (c * group + j) * hd + d]);
    }
    Qs[r * ldq + d] = val;
  }

  const int my_pair = pair0 + row;
  const bool row_valid = my_pair < n_pairs;
  const int my_t = row_valid ? my_pair / group : 0;
  const int my_limit = ctx + my_t;                                    // last visible key
  const int my_first = p.window > 0 ? max(0, my_limit - p.window + 1) : 0;
  const int my_chunk0 = p.chunk > 0 ? (my_limit / p.chunk) * p.chunk : 0;
  const int cv = c / (p.n_kv_heads / p.n_v_heads);
  const int my_head = c * group + (row_valid ? my_pair - my_t * group : 0);
  const float* my_bias = (p.score_bias != nullptr && row_valid) ? p.score_bias + (size_t)my_head * p.bias_dists : nullptr;
  const float my_scale = p.head_scale != nullptr ? p.scale * p.head_scale[my_head] : p.scale;

  const int last_pair = min(pair0 + AG_ROWS, n_pairs) - 1;
  const int key_end = ctx + last_pair / group + 1;                     // keys [.., key_end) matter to the tile
  int key_begin = 0;
  if (p.window > 0) {
    const int first_t = pair0 / group;
    key_begin = max(0, ctx + first_t - p.window + 1);
    key_begin = (key_begin / AG_KEYS) * AG_KEYS;
  }
  if (p.chunk > 0) {
    // rows of a tile ascend in position: the first row's chunk starts first
    const int c0 = ((ctx + pair0 / group) / p.chunk) * p.chunk;
    key_begin = max(key_begin, (c0 / AG_KEYS) * AG_KEYS);
  }
  // with kept first keys the walk starts with their tiles and then jumps to the window's first tile
  const int keep = p.window > 0 ? p.keep_first : 0;
  const int keep_end = ((keep + AG_KEYS - 1) / AG_KEYS) * AG_KEYS;

  float acc[AG_MAX_ACC];
#pragma unroll
  for (int i = 0; i < AG_MAX_ACC; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const int n_acc = (hdv + 7) >> 3;       // the last one of a value size that is no multiple of 8 is partly idle

  for (int kt = keep > 0 ? 0 : key_begin; kt < key_end; kt += AG_KEYS) {
    if (kt >= keep_end && kt < key_begin) kt = key_begin;       // (both multiples of the tile)
    __syncthreads();  // previous tile fully consumed (and Qs staged, first time)
    for (int idx = tid; idx < AG_KEYS * hd; idx += AG_THREADS) {
      const int kk = idx / hd, d = idx - kk * hd;
      const int kp = kt + kk;
      float kv = 0.f;
      if (kp < key_end) {
        const int page = IE_PAGE(table[kp / p.page_size]);
        if (page >= 0)
          kv = to_f32(kpool[(((size_t)page * p.n_kv_heads + c) * p.page_size + (kp % p.page_size)) * hd + d]);
      }
      Ks[kk * ldq + d] = kv;
    }
    for (int idx = tid; idx < AG_KEYS * hdv; idx += AG_THREADS) {
      const int kk = idx / hdv, d = idx - kk * hdv;
      const int kp = kt + kk;
      float vv = 0.f;
      if (kp < key_end) {
        const int page = IE_PAGE(table[kp / p.page_size]);
        if (page >= 0)
          vv = to_f32(vpool[(((size_t)page * p.n_v_heads + cv) * p.page_size + (kp % p.page_size)) * p.v_row + d]);
      }
      Vs[kk * hdv + d] = vv;
    }
    __syncthreads();

    // scores of this thread: keys sub, sub+8, sub+16, sub+24 of its row
    float s[4];
    float tile_max = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int kk = sub + 8 * jj;
      const int kp = kt + kk;
      float dot = 0.f;
      const float* qr = Qs + row * ldq;
      const float* kr = Ks + kk * ldq;
      for (int d = 0; d < hd; ++d) dot += qr[d] * kr[d];
      const bool visible = row_valid && kp <= my_limit && kp >= my_chunk0 && (kp >= my_first || kp < keep);
      float sc = dot * my_scale;
      if (visible && my_bias != nullptr) sc += my_bias[min(my_limit - kp, p.bias_dists - 1)];
      s[jj] = visible ? sc : -INFINITY;
      tile_max = fmaxf(tile_max, s[jj]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
    const float m_new = fmaxf(m_run, tile_max);
    float alpha = 1.f, psum = 0.f;
    if (m_new == -INFINITY) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) Ps[row * (AG_KEYS + 1) + sub + 8 * jj] = 0.f;
    } else {
      alpha = expf(m_run - m_new);  // exp(-inf) = 0 on the first tile with a visible key
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float e = expf(s[jj] - m_new);
        Ps[row * (AG_KEYS + 1) + sub + 8 * jj] = e;
        psum += e;
      }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l_run = l_run * alpha + psum;
    m_run = m_new;
    __syncthreads();

    // out accumulators: dims sub, sub+8, ... of this row
    const float* pr_ = Ps + row * (AG_KEYS + 1);
#pragma unroll
    for (int i = 0; i < AG_MAX_ACC; ++i) {
      if (i < n_acc && sub + 8 * i < hdv) {
        float a = acc[i] * alpha;
        const float* vcol = Vs + sub + 8 * i;
#pragma unroll 8
        for (int kk = 0; kk < AG_KEYS; ++kk) a += pr_[kk] * vcol[kk * hdv];
        acc[i] = a;
      }
    }
  }

  if (row_valid) {
    const int j = my_pair - my_t * group;
    T* o = (T*)p.out + (size_t)(q0 + my_t) * p.out_stride + (c * group + j) * hdv;
    const float inv = inv_with_sink(l_run, m_run, p.sink, my_head, p.out_scale);
#pragma unroll
    for (int i = 0; i < AG_MAX_ACC; ++i)
      if (i < n_acc && sub + 8 * i < hdv) o[sub + 8 * i] = from_f32<T>(acc[i] * inv);
  }
}

extern "C" int ie_attention_general(const void* q, void* out, const void* kpool, const void* vpool,
                                    const int* block_table, const int* q_start, const int* ctx_before,
                                    const int* work_req, const int* work_pair0, int q_stride, int out_stride,
                                    int table_stride, int n_work, int n_heads, int n_kv_heads, int hd,
                                    int page_size, int window, float scale, int act_dtype, const float* score_bias,
                                    int bias_dists, const float* head_scale, int hd_v, int keep_first,
                                    float out_scale, int chunk, int n_v_heads, int v_row, const float* sink,
                                    cudaStream_t stream) {
  if (n_work <= 0) return IE_OK;
  if (hd_v <= 0) hd_v = hd;
  if (hd <= 0 || hd > 8 * AG_MAX_ACC || hd_v > 8 * AG_MAX_ACC) return IE_BAD_SIZE;
  if (n_kv_heads <= 0 || n_heads % n_kv_heads) return IE_BAD_SIZE;
  if (score_bias != nullptr && bias_dists <= 0) return IE_BAD_SIZE;
  if (n_v_heads <= 0) n_v_heads = n_kv_heads;
  if (v_row <= 0) v_row = hd_v;
  if (n_kv_heads % n_v_heads || v_row < hd_v || chunk < 0 || (chunk > 0 && keep_first > 0)) return IE_BAD_SIZE;
  AttnGeneralParams p;
  p.chunk = chunk; p.n_v_heads = n_v_heads; p.v_row = v_row; p.sink = sink;
  p.q = q; p.out = out; p.kpool = kpool; p.vpool = vpool; p.block_table = block_table;
  p.q_start = q_start; p.ctx_before = ctx_before; p.work_req = work_req; p.work_pair0 = work_pair0;
  p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride;
  p.n_work = n_work; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.hd = hd; p.page_size = page_size;
  p.window = window; p.scale = scale; p.score_bias = score_bias; p.bias_dists = bias_dists;
  p.head_scale = head_scale; p.hd_v = hd_v; p.keep_first = keep_first > 0 ? keep_first : 0; p.out_scale = out_scale;
  const size_t smem = sizeof(float) * ((size_t)AG_ROWS * (hd + 1) + (size_t)AG_KEYS * (hd + 1) +
                                       (size_t)AG_KEYS * hd_v + (size_t)AG_ROWS * (AG_KEYS + 1));
  dim3 grid(n_work, n_kv_heads);
  cudaError_t e;
  if (act_dtype == IE_F32) {
    e = cudaFuncSetAttribute(attention_general_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch_k(attention_general_kernel<float>, grid, AG_THREADS, smem, stream, p);
  } else if (act_dtype == IE_BF16) {
    e = cudaFuncSetAttribute(attention_general_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch_k(attention_general_kernel<bf16>, grid, AG_THREADS, smem, stream, p);
  }
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ few rows a request (decode steps)
// The tile kernel above gives a (request, kv head) one block, which for a request that brings a single token walks
// all its keys alone.  This one gives every (token, query head) of a request that brings at most `max_rows` (token,
// head-in-group) rows a block of sixteen warps.  A warp takes the visible keys (the kept first keys, then the window's)
// 32 at a time, warp w the groups w, w + 16, ...: each lane forms the score of ONE key (the query is read from shared
// memory, the key's row in 16-byte pieces where the sizes allow), the 32 scores meet the running maximum and sum
// through two warp reductions, and then the lanes turn to the output's dimensions and add the 32 values' rows, the
// weights passed round by shuffles, 16, 8 or 4 rows on their way together (the kernel is built for 2, 4 and 8 values
// a lane: value heads up to 64, 128, 256).  The warps' results are merged in shared memory in warp order.  Same
// arithmetic as above (float32 scores, weights and sums), same options.  Requests with more rows are left to the
// tile kernel, whose work list then names only those.
#define AR_WARPS 16
#define AR_MAX_PER_LANE 8   // head sizes up to 256

template <typename T>
__device__ __forceinline__ float key_dot(const T* __restrict__ krow, const float* __restrict__ qs, int hd) {
  float s0 = 0.f, s1 = 0.f;
  if (sizeof(T) == 2 && (hd & 7) == 0 && (((uintptr_t)krow) & 15) == 0) {
    for (int d = 0; d < hd; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float4 qa = *reinterpret_cast<const float4*>(qs + d), qb = *reinterpret_cast<const float4*>(qs + d + 4);
      const float2 k0 = __bfloat1622float2(h[0]), k1 = __bfloat1622float2(h[1]), k2 = __bfloat1622float2(h[2]),
                   k3 = __bfloat1622float2(h[3]);
      s0 = fmaf(qa.x, k0.x, s0); s1 = fmaf(qa.y, k0.y, s1); s0 = fmaf(qa.z, k1.x, s0); s1 = fmaf(qa.w, k1.y, s1);
      s0 = fmaf(qb.x, k2.x, s0); s1 = fmaf(qb.y, k2.y, s1); s0 = fmaf(qb.z, k3.x, s0); s1 = fmaf(qb.w, k3.y, s1);
    }
  } else if (sizeof(T) == 4 && (hd & 3) == 0 && (((uintptr_t)krow) & 15) == 0) {
    for (int d = 0; d < hd; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(krow + d);
      const float4 qa = *reinterpret_cast<const float4*>(qs + d);
      s0 = fmaf(qa.x, kv.x, s0); s1 = fmaf(qa.y, kv.y, s1); s0 = fmaf(qa.z, kv.z, s0); s1 = fmaf(qa.w, kv.w, s1);
    }
  } else {
    for (int d = 0; d < hd; ++d) s0 = fmaf(qs[d], to_f32(krow[d]), s0);
  }
  return s0 + s1;
}

template <typename T, int PL>
__global__ void __launch_bounds__(AR_WARPS * 32) attention_rows_kernel(AttnGeneralParams p, int n_requests, int max_rows) {
  constexpr int VU = 32 / PL;                      // value rows in flight
  __shared__ float s_m[AR_WARPS], s_l[AR_WARPS];
  extern __shared__ __align__(16) float s_dyn[];   // the query [hd rounded up to 4], then [AR_WARPS][hd_v]
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x, head = blockIdx.y;
  int lo = 0, hi = n_requests;                     // the request r with q_start[r] <= n < q_start[r + 1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.q_start[mid] <= n) lo = mid; else hi = mid;
  }
  const int r_id = lo;
  const int group = p.n_heads / p.n_kv_heads;
  const int q0 = p.q_start[r_id], q_len = p.q_start[r_id + 1] - q0;
  if (q_len * group > max_rows) return;            // the tile kernel's
  const int hd = p.hd, hdv = p.hd_v;
  float* qs = s_dyn;
  float* s_acc = s_dyn + ((hd + 3) & ~3);
  const int c = head / group;
  const int limit = p.ctx_before[r_id] + (n - q0);                       // last visible key
  int first = p.window > 0 ? max(0, limit - p.window + 1) : 0;
  if (p.chunk > 0) first = max(first, (limit / p.chunk) * p.chunk);
  const int cv = c / (p.n_kv_heads / p.n_v_heads);
  const int n_keep = p.window > 0 ? min(p.keep_first, first) : 0;         // kept keys that the window does not hold anyway
  const int n_vis = n_keep + (limit - first + 1);
  const int* table = p.block_table + (size_t)r_id * p.table_stride;
  const T* kpool = (const T*)p.kpool;
  const T* vpool = (const T*)p.vpool;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* qrow = (const T*)p.q + (size_t)n * p.q_stride + head * hd;
  for (int d = threadIdx.x; d < hd; d += AR_WARPS * 32) qs[d] = to_f32(qrow[d]);
  __syncthreads();
  float acc[PL];
#pragma unroll
  for (int j = 0; j < PL; ++j) acc[j] = 0.f;
  const float my_scale = p.head_scale != nullptr ? p.scale * p.head_scale[head] : p.scale;
  const float* my_bias = p.score_bias != nullptr ? p.score_bias + (size_t)head * p.bias_dists : nullptr;
  float m_run = -INFINITY, l_run = 0.f;
  for (int i0 = warp * 32; i0 < n_vis; i0 += AR_WARPS * 32) {
    const int idx = i0 + lane;
    float sc = -INFINITY;
    long long at = -1, vat_mine = -1;              // this lane's key: its row in the key pool and in the value pool
    if (idx < n_vis) {
      const int kp = idx < n_keep ? idx : first + (idx - n_keep);
      const int page = IE_PAGE(table[kp / p.page_size]);
      if (page >= 0) {
        at = ((long long)page * p.n_kv_heads + c) * p.page_size + (kp % p.page_size);
        vat_mine = ((long long)page * p.n_v_heads + cv) * p.page_size + (kp % p.page_size);
        sc = key_dot(kpool + at * hd, qs, hd) * my_scale;
        if (my_bias != nullptr) sc += my_bias[min(limit - kp, p.bias_dists - 1)];
      }
    }
    const float m_new = fmaxf(m_run, warp_max(sc));
    if (m_new == -INFINITY) continue;              // (the same in every lane)
    const float alpha = expf(m_run - m_new);       // exp(-inf) = 0 the first time
    const float e = at >= 0 ? expf(sc - m_new) : 0.f;
    l_run = l_run * alpha + warp_sum(e);
    m_run = m_new;
#pragma unroll
    for (int j = 0; j < PL; ++j) acc[j] *= alpha;
    const int n_here = min(32, n_vis - i0);
    for (int kk0 = 0; kk0 < n_here; kk0 += VU) {    // VU keys' value rows on their way together
      float w[VU];
      T vals[VU][PL];
#pragma unroll
      for (int u = 0; u < VU; ++u) {
        const int kk = (kk0 + u) & 31;
        const float wk = __shfl_sync(0xffffffffu, e, kk);
        const long long vat = __shfl_sync(0xffffffffu, vat_mine, kk);
        const bool live = kk0 + u < n_here && vat >= 0;
        w[u] = live ? wk : 0.f;
        const T* vrow = vpool + (live ? vat : 0) * p.v_row;
#pragma unroll
        for (int j = 0; j < PL; ++j) {
          const int d = lane + 32 * j;
          vals[u][j] = (d < hdv && live) ? vrow[d] : from_f32<T>(0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < VU; ++u)
#pragma unroll
        for (int j = 0; j < PL; ++j) acc[j] = fmaf(w[u], to_f32(vals[u][j]), acc[j]);
    }
  }
  if (lane == 0) {
    s_m[warp] = m_run;
    s_l[warp] = l_run;
  }
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const int d = lane + 32 * j;
    if (d < hdv) s_acc[warp * hdv + d] = acc[j];
  }
  __syncthreads();
  float m_all = -INFINITY;
#pragma unroll
  for (int w = 0; w < AR_WARPS; ++w) m_all = fmaxf(m_all, s_m[w]);
  float l_all = 0.f;
#pragma unroll
  for (int w = 0; w < AR_WARPS; ++w) l_all += s_m[w] == -INFINITY ? 0.f : s_l[w] * expf(s_m[w] - m_all);
  const float inv = inv_with_sink(l_all, m_all, p.sink, head, p.out_scale);
  T* o = (T*)p.out + (size_t)n * p.out_stride + head * hdv;
  for (int d = threadIdx.x; d < hdv; d += AR_WARPS * 32) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < AR_WARPS; ++w)
      if (s_m[w] != -INFINITY) total = fmaf(s_acc[w * hdv + d], expf(s_m[w] - m_all), total);
    o[d] = from_f32<T>(total * inv);
  }
}

extern "C" int ie_attention_rows(const void* q, void* out, const void* kpool, const void* vpool, const int* block_table,
                                 const int* q_start, const int* ctx_before, int q_stride, int out_stride, int table_stride,
                                 int n_tokens, int n_requests, int max_rows, int n_heads, int n_kv_heads, int hd,
                                 int page_size, int window, float scale, int act_dtype, const float* score_bias,
                                 int bias_dists, const float* head_scale, int hd_v, int keep_first, float out_scale,
                                 int chunk, int n_v_heads, int v_row, const float* sink, cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return IE_OK;
  if (hd_v <= 0) hd_v = hd;
  if (hd <= 0 || hd > 32 * AR_MAX_PER_LANE || hd_v > 32 * AR_MAX_PER_LANE) return IE_BAD_SIZE;
  if (n_kv_heads <= 0 || n_heads % n_kv_heads || n_heads > 65535) return IE_BAD_SIZE;
  if (score_bias != nullptr && bias_dists <= 0) return IE_BAD_SIZE;
  if (n_v_heads <= 0) n_v_heads = n_kv_heads;
  if (v_row <= 0) v_row = hd_v;
  if (n_kv_heads % n_v_heads || v_row < hd_v || chunk < 0 || (chunk > 0 && keep_first > 0)) return IE_BAD_SIZE;
  AttnGeneralParams p;
  p.chunk = chunk; p.n_v_heads = n_v_heads; p.v_row = v_row; p.sink = sink;
  p.q = q; p.out = out; p.kpool = kpool; p.vpool = vpool; p.block_table = block_table;
  p.q_start = q_start; p.ctx_before = ctx_before; p.work_req = nullptr; p.work_pair0 = nullptr;
  p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride;
  p.n_work = 0; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.hd = hd; p.page_size = page_size;
  p.window = window; p.scale = scale; p.score_bias = score_bias; p.bias_dists = bias_dists;
  p.head_scale = head_scale; p.hd_v = hd_v; p.keep_first = keep_first > 0 ? keep_first : 0; p.out_scale = out_scale;
  const size_t smem = sizeof(float) * (((size_t)hd + 3) / 4 * 4 + AR_WARPS * (size_t)hd_v);
  dim3 grid(n_tokens, n_heads);
  const int pl = hd_v <= 64 ? 2 : (hd_v <= 128 ? 4 : 8);
#define AR_GO(T, PL) return launch_k(attention_rows_kernel<T, PL>, grid, AR_WARPS * 32, smem, stream, p, n_requests, max_rows)
  if (act_dtype == IE_F32) {
    if (pl == 2) AR_GO(float, 2);
    if (pl == 4) AR_GO(float, 4);
    AR_GO(float, 8);
  }
  if (act_dtype == IE_BF16) {
    if (pl == 2) AR_GO(bf16, 2);
    if (pl == 4) AR_GO(bf16, 4);
    AR_GO(bf16, 8);
  }
#undef AR_GO
  return IE_BAD_DTYPE;
}

IE_CHECK_API(attention_general)
