// Paged causal attention for prompt portions on tensor cores with float32 scores, one (key head size, value head size)
// per build (-DIE_AW_DK, -DIE_AW_DV: multiples of 16 up to 256, each its own).  It serves layers whose scores, weights
// and sums are to be float32 and whose shape the other tensor-core kernels do not take: values of another size than the
// keys, several key heads over one value head (two score maps a head), values that are the first dimensions of the key
// rows (a compressed key/value vector stored once, read by every query head), a mask by chunks of positions.
//
//   out[t, h] = sum_j w_j v_j / sum_j w_j,   w_j = exp(scale * q[t, h] . k_j - m)   over the visible keys j
//   visible: j <= p = ctx_before + t,  j > p - window (if set),  j >= floor(p / chunk) * chunk (if set)
//
// A block of four warps takes one (request, key head) and a tile of 64 (token, head-in-group) pairs, so the query heads
// that share a key head share every key tile that is loaded.  Keys are walked in tiles at absolute multiples of the
// tile, ascending, double-buffered through cp.async.  q k^T is mma.sync m16n8k16 on the bfloat16 operands as they are
// (their products are exact in float32, the sums are float32); maxima, exponentials and sums are float32; a weight
// meets the values as TWO bfloat16 terms (its rounding and what that left out), both through the tensor cores into
// float32 accumulators, so it carries 16 bits of mantissa.
#include "common.cuh"

#ifndef IE_AW_DK
#define IE_AW_DK 64
#endif
#ifndef IE_AW_DV
#define IE_AW_DV 64
#endif

namespace {

constexpr int DK = IE_AW_DK, DV = IE_AW_DV;
static_assert(DK > 0 && DV > 0 && DK <= 256 && DV <= 256 && DK % 16 == 0 && DV % 16 == 0, "head sizes: multiples of 16 up to 256");
constexpr int BM = 64;                                // rows of a tile: 16 a warp
constexpr int BN = (DK + DV <= 256) ? 64 : 32;        // keys of a tile
constexpr int THREADS = 128;
constexpr int LDK = DK + 8, LDV = DV + 8;             // a row of shared memory: an odd number of 16-byte pieces
constexpr int KSTEPS = DK / 16, NT_S = BN / 8, NT_O = DV / 8;
constexpr int KC = DK / 8, VC = DV / 8;               // 16-byte pieces of a row
constexpr float LOG2E = 1.4426950408889634f;

struct WideParams {
  const bf16* q;
  bf16* out;
  const bf16* kpool;
  const bf16* vpool;
  const int* block_table;
  const int* q_start;
  const int* ctx_before;
  const int* work_req;
  const int* work_pair0;
  int q_stride, out_stride, table_stride;
  int n_heads, n_kv_heads, page_size, window, chunk;
  int n_v_heads;   // key head c reads value head c / (n_kv_heads / n_v_heads)
  int v_row;       // elements between two value rows of the value pool
  int alias;       // the values are the first DV dimensions of the key rows: the key tile is the value tile
  float scale_log2;
  // without a work list (work_req null): block x is tile x % tiles of request x / tiles, and only requests that bring
  // at most max_rows (token, head-in-group) pairs take part (decode tokens; the others are a work list's)
  int tiles, max_rows;
  // n_splits > 1: block z takes the keys [first + z * split_keys, first + (z + 1) * split_keys) of its tile's range
  // (split_keys a multiple of the key tile) and leaves sums, maxima and unnormalised outputs for the merge kernel
  int n_splits, split_keys;
  const float* sink;  // [n_heads] or null: the denominator of head h also holds exp(sink[h]), a logit that weighs nothing
  float* part_o;   // [blocks x, key heads, splits, BM, DV]
  float* part_ml;  // [blocks x, key heads, splits, BM, 2]
};

__device__ __forceinline__ void cp16(void* dst, const void* src) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(unsigned (&r)[4], const bf16* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4_t(unsigned (&r)[4], const bf16* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack2(float x, float y) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);   // x in the low half
  return *reinterpret_cast<const unsigned*>(&h);
}
// a weight in two bfloat16 terms: hi = round(p), lo = round(p - hi)
__device__ __forceinline__ void split2(float x, float y, unsigned& hi, unsigned& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  const float2 hf = __bfloat1622float2(h);
  hi = *reinterpret_cast<const unsigned*>(&h);
  lo = pack2(x - hf.x, y - hf.y);
}

// keys kt .. kt + BN - 1 of a request's key head c (and of value head cv) into one buffer pair; keys from key_end on and
// pages that are not held read as zeros
__device__ __forceinline__ void load_tile(const WideParams& p, bf16* Ks, bf16* Vs, int kt, int key_end, const int* table,
                                          int c, int cv, int tid) {
  for (int idx = tid; idx < BN * KC; idx += THREADS) {
    const int kk = idx / KC, ch = idx - kk * KC;
    const int kp = kt + kk;
    bf16* dst = Ks + kk * LDK + ch * 8;
    int page = -1;
    if (kp < key_end) page = IE_PAGE(table[kp / p.page_size]);
    if (page >= 0)
      cp16(dst, p.kpool + (((size_t)page * p.n_kv_heads + c) * p.page_size + (kp % p.page_size)) * DK + ch * 8);
    else
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (p.alias) return;
  for (int idx = tid; idx < BN * VC; idx += THREADS) {
    const int kk = idx / VC, ch = idx - kk * VC;
    const int kp = kt + kk;
    bf16* dst = Vs + kk * LDV + ch * 8;
    int page = -1;
    if (kp < key_end) page = IE_PAGE(table[kp / p.page_size]);
    if (page >= 0)
      cp16(dst, p.vpool + (((size_t)page * p.n_v_heads + cv) * p.page_size + (kp % p.page_size)) * p.v_row + ch * 8);
    else
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// 1 / (l + the sink's term) for a row whose sum l was formed at the maximum m (both in the exponent's base-2 units)
__device__ __forceinline__ float wide_inv(float l, float m, const float* sink, int head) {
  if (sink == nullptr || m == -INFINITY) return l > 0.f ? 1.f / l : 0.f;
  const float sk = sink[head] * LOG2E;
  const float m2 = fmaxf(m, sk);
  const float f = exp2f(m - m2);
  return f / (l * f + exp2f(sk - m2));
}

__global__ void __launch_bounds__(THREADS) attention_wide_kernel(WideParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_trigger();
  pdl_wait();
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);   // [BM][LDK]
  bf16* Kbuf = Qs + BM * LDK;                     // [2][BN][LDK]
  bf16* Vbuf = Kbuf + 2 * BN * LDK;               // [2][BN][LDV] (unused when the values are in the keys)

  const int r_id = p.work_req != nullptr ? p.work_req[blockIdx.x] : (int)blockIdx.x / p.tiles;
  const int pair0 = p.work_req != nullptr ? p.work_pair0[blockIdx.x] : ((int)blockIdx.x % p.tiles) * BM;
  const int c = blockIdx.y;
  const int group = p.n_heads / p.n_kv_heads;
  const int cv = c / (p.n_kv_heads / p.n_v_heads);
  const int q0 = p.q_start[r_id];
  const int n_pairs = (p.q_start[r_id + 1] - q0) * group;
  if (p.work_req == nullptr && (n_pairs > p.max_rows || pair0 >= n_pairs)) return;
  const int ctx = p.ctx_before[r_id];
  const int* table = p.block_table + (size_t)r_id * p.table_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;

  // the tile's queries
  for (int idx = tid; idx < BM * KC; idx += THREADS) {
    const int r = idx / KC, ch = idx - r * KC;
    const int pr = pair0 + r;
    bf16* dst = Qs + r * LDK + ch * 8;
    if (pr < n_pairs) {
      const int t = pr / group, j = pr - t * group;
      cp16(dst, p.q + (size_t)(q0 + t) * p.q_stride + (size_t)(c * group + j) * DK + ch * 8);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }

  // what this thread's two rows (g and g + 8 of its warp's sixteen) may see: keys lo .. limit
  int limit[2], lo[2], pr_[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    pr_[h] = pair0 + warp * 16 + g + 8 * h;
    if (pr_[h] < n_pairs) {
      limit[h] = ctx + pr_[h] / group;
      int first = p.window > 0 ? max(0, limit[h] - p.window + 1) : 0;
      if (p.chunk > 0) first = max(first, (limit[h] / p.chunk) * p.chunk);
      lo[h] = first;
    } else {
      limit[h] = -1;
      lo[h] = 0;
    }
  }
  const int last_pair = min(pair0 + BM, n_pairs) - 1;
  const int key_end = ctx + last_pair / group + 1;
  int key_begin = 0;                                 // rows of a tile ascend in position: the first row starts first
  {
    const int p_first = ctx + pair0 / group;
    if (p.window > 0) key_begin = max(0, p_first - p.window + 1);
    if (p.chunk > 0) key_begin = max(key_begin, (p_first / p.chunk) * p.chunk);
    key_begin = (key_begin / BN) * BN;
  }

  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int ldv = p.alias ? LDK : LDV;

  int k_lo = key_begin, k_hi = key_end;
  if (p.n_splits > 1) {
    k_lo = key_begin + (int)blockIdx.z * p.split_keys;
    k_hi = min(key_end, k_lo + p.split_keys);
  }
  if (k_lo < k_hi) load_tile(p, Kbuf, Vbuf, k_lo, key_end, table, c, cv, tid);
  cp_commit();
  int buf = 0;
  for (int kt = k_lo; kt < k_hi; kt += BN, buf ^= 1) {
    const bool more = kt + BN < k_hi;
    if (more) {
      load_tile(p, Kbuf + (buf ^ 1) * BN * LDK, Vbuf + (buf ^ 1) * BN * LDV, kt + BN, key_end, table, c, cv, tid);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    const bf16* Kt = Kbuf + buf * BN * LDK;
    const bf16* Vt = p.alias ? Kt : Vbuf + buf * BN * LDV;

    float s[NT_S][4];
#pragma unroll
    for (int i = 0; i < NT_S; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      unsigned a[4];
      ldsm4(a, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < NT_S / 2; ++np) {
        unsigned b[4];
        ldsm4(b, Kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
        mma16816(s[2 * np], a, b[0], b[1]);
        mma16816(s[2 * np + 1], a, b[2], b[3]);
      }
    }

    // mask, scale, running maximum (exponent units: scale * log2 e is in the multiplier)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int kp = kt + nt * 8 + 2 * t4 + (e & 1);
        const bool vis = kp >= lo[h] && kp <= limit[h];
        const float v = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
        s[nt][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      alpha[h] = m_new == -INFINITY ? 1.f : exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const float pv = m_run[h] == -INFINITY ? 0.f : exp2f(s[nt][e] - m_run[h]);
        s[nt][e] = pv;
        psum[h] += pv;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + psum[h];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }

    // weights times values, sixteen keys a step
#pragma unroll
    for (int k2 = 0; k2 < BN / 16; ++k2) {
      unsigned ah[4], al[4];
      split2(s[2 * k2][0], s[2 * k2][1], ah[0], al[0]);
      split2(s[2 * k2][2], s[2 * k2][3], ah[1], al[1]);
      split2(s[2 * k2 + 1][0], s[2 * k2 + 1][1], ah[2], al[2]);
      split2(s[2 * k2 + 1][2], s[2 * k2 + 1][3], ah[3], al[3]);
#pragma unroll
      for (int dp = 0; dp < NT_O / 2; ++dp) {
        unsigned b[4];
        ldsm4_t(b, Vt + (k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + dp * 16 + (lane >> 4) * 8);
        mma16816(o[2 * dp], ah, b[0], b[1]);
        mma16816(o[2 * dp], al, b[0], b[1]);
        mma16816(o[2 * dp + 1], ah, b[2], b[3]);
        mma16816(o[2 * dp + 1], al, b[2], b[3]);
      }
    }
    __syncthreads();   // the tile is used up before the load after next overwrites it
  }
  cp_wait<0>();

  if (p.n_splits > 1) {
    const size_t part = ((size_t)blockIdx.x * p.n_kv_heads + c) * p.n_splits + blockIdx.z;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float l = l_run[h];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (pr_[h] >= n_pairs) continue;
      const size_t row = part * BM + warp * 16 + g + 8 * h;
      if (t4 == 0) {
        p.part_ml[row * 2] = m_run[h];
        p.part_ml[row * 2 + 1] = l;
      }
      float* dst = p.part_o + row * DV + 2 * t4;
#pragma unroll
      for (int i = 0; i < NT_O; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
    }
    return;
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = l_run[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (pr_[h] >= n_pairs) continue;
    const int t = pr_[h] / group, j = pr_[h] - t * group;
    const float inv = wide_inv(l, m_run[h], p.sink, c * group + j);
    bf16* dst = p.out + (size_t)(q0 + t) * p.out_stride + (size_t)(c * group + j) * DV + 2 * t4;
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
  }
}

// the splits of a tile become its output rows: out = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), m = max_s m_s.
// A warp a row (block z takes rows 4 z .. 4 z + 3 of the tile): its lanes find m over the splits together, then walk the
// splits with the row's values spread over the lanes, so every load of a partial output is one contiguous piece.
constexpr int MERGE_ROWS = THREADS / 32;
constexpr int MERGE_SLOTS = (DV + 63) / 64;           // pairs of values a lane holds

__global__ void __launch_bounds__(THREADS) attention_wide_merge_kernel(WideParams p) {
  pdl_trigger();
  pdl_wait();
  const int r_id = (int)blockIdx.x / p.tiles, pair0 = ((int)blockIdx.x % p.tiles) * BM;
  const int c = blockIdx.y;
  const int group = p.n_heads / p.n_kv_heads;
  const int q0 = p.q_start[r_id];
  const int n_pairs = (p.q_start[r_id + 1] - q0) * group;
  if (n_pairs > p.max_rows || pair0 >= n_pairs) return;
  const int rows = min(BM, n_pairs - pair0);
  const int lane = threadIdx.x & 31;
  const int r = (int)blockIdx.z * MERGE_ROWS + ((int)threadIdx.x >> 5);
  if (r >= rows) return;                              // (the whole warp)
  const size_t part0 = ((size_t)blockIdx.x * p.n_kv_heads + c) * p.n_splits;
  float m_all = -INFINITY;
  for (int s = lane; s < p.n_splits; s += 32) m_all = fmaxf(m_all, p.part_ml[((part0 + s) * BM + r) * 2]);
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, k));
  float l_all = 0.f;
  float2 acc[MERGE_SLOTS];
#pragma unroll
  for (int i = 0; i < MERGE_SLOTS; ++i) acc[i] = make_float2(0.f, 0.f);
  if (m_all != -INFINITY) {
#pragma unroll 4
    for (int s = 0; s < p.n_splits; ++s) {
      const size_t row = (part0 + s) * BM + r;
      const float2 ml = *reinterpret_cast<const float2*>(p.part_ml + row * 2);
      const float w = ml.x == -INFINITY ? 0.f : exp2f(ml.x - m_all);
      l_all = fmaf(ml.y, w, l_all);
#pragma unroll
      for (int i = 0; i < MERGE_SLOTS; ++i) {
        const int d = (i * 32 + lane) * 2;
        if (d < DV && w != 0.f) {
          const float2 v = *reinterpret_cast<const float2*>(p.part_o + row * DV + d);
          acc[i].x = fmaf(v.x, w, acc[i].x);
          acc[i].y = fmaf(v.y, w, acc[i].y);
        }
      }
    }
  }
  const int pr = pair0 + r;
  const int t = pr / group, j = pr - t * group;
  const float inv = wide_inv(l_all, m_all, p.sink, c * group + j);
  bf16* dst = p.out + (size_t)(q0 + t) * p.out_stride + (size_t)(c * group + j) * DV;
#pragma unroll
  for (int i = 0; i < MERGE_SLOTS; ++i) {
    const int d = (i * 32 + lane) * 2;
    if (d < DV) *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(acc[i].x * inv, acc[i].y * inv);
  }
}

}  // namespace

extern "C" int ie_attention_wide_key_dim() { return DK; }
extern "C" int ie_attention_wide_value_dim() { return DV; }
extern "C" int ie_attention_wide_rows() { return BM; }
extern "C" int ie_attention_wide_keys() { return BN; }

static int wide_params(WideParams& p, const void* q, void* out, const void* kpool, const void* vpool, const int* block_table,
                       const int* q_start, const int* ctx_before, int q_stride, int out_stride, int table_stride, int n_heads,
                       int n_kv_heads, int page_size, int window, float scale, int chunk, int n_v_heads, int v_row,
                       const float* sink) {
  if (n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 || window < 0 || chunk < 0) return IE_BAD_SIZE;
  if (n_v_heads <= 0) n_v_heads = n_kv_heads;
  if (v_row <= 0) v_row = DV;
  if (n_kv_heads % n_v_heads || v_row < DV) return IE_BAD_SIZE;
  // cp.async moves 16 bytes: rows of q and of the pools start on such a boundary, the output takes pairs
  if (((uintptr_t)q & 15) || ((uintptr_t)kpool & 15) || ((uintptr_t)vpool & 15) || ((uintptr_t)out & 3) || (q_stride & 7) ||
      (out_stride & 1) || (v_row & 7))
    return IE_BAD_ALIGN;
  p.q = (const bf16*)q; p.out = (bf16*)out; p.kpool = (const bf16*)kpool; p.vpool = (const bf16*)vpool;
  p.block_table = block_table; p.q_start = q_start; p.ctx_before = ctx_before; p.work_req = nullptr; p.work_pair0 = nullptr;
  p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size; p.window = window; p.chunk = chunk;
  p.n_v_heads = n_v_heads; p.v_row = v_row; p.sink = sink;
  p.alias = (vpool == kpool && v_row == DK && n_v_heads == n_kv_heads && DV <= DK) ? 1 : 0;
  p.scale_log2 = scale * LOG2E;
  p.tiles = 1; p.max_rows = 0; p.n_splits = 1; p.split_keys = 0; p.part_o = nullptr; p.part_ml = nullptr;
  return IE_OK;
}

static size_t wide_smem(const WideParams& p) {
  return sizeof(bf16) * ((size_t)BM * LDK + 2 * (size_t)BN * LDK + (p.alias ? 0 : 2 * (size_t)BN * LDV));
}

extern "C" int ie_attention_wide(const void* q, void* out, const void* kpool, const void* vpool, const int* block_table,
                                 const int* q_start, const int* ctx_before, const int* work_req, const int* work_pair0,
                                 int q_stride, int out_stride, int table_stride, int n_work, int n_heads, int n_kv_heads,
                                 int page_size, int window, float scale, int chunk, int n_v_heads, int v_row,
                                 const float* sink, cudaStream_t stream) {
  if (n_work <= 0) return IE_OK;
  if (work_req == nullptr || work_pair0 == nullptr) return IE_BAD_SIZE;
  WideParams p;
  const int rc = wide_params(p, q, out, kpool, vpool, block_table, q_start, ctx_before, q_stride, out_stride, table_stride,
                             n_heads, n_kv_heads, page_size, window, scale, chunk, n_v_heads, v_row, sink);
  if (rc != IE_OK) return rc;
  p.work_req = work_req; p.work_pair0 = work_pair0;
  const size_t smem = wide_smem(p);
  cudaError_t e = cudaFuncSetAttribute(attention_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return launch_k(attention_wide_kernel, dim3(n_work, n_kv_heads), THREADS, smem, stream, p);
}

// floats of scratch that ie_attention_wide_small needs
extern "C" long long ie_attention_wide_small_scratch(int n_requests, int max_rows, int n_kv_heads, int n_splits) {
  const long long tiles = (max_rows + BM - 1) / BM;
  return n_splits > 1 ? (long long)n_requests * tiles * n_kv_heads * n_splits * BM * (DV + 2) : 0;
}

// The requests of the step that bring at most max_rows (token, head-in-group) pairs (decode tokens, as a rule), without
// a work list: every such request's keys are cut into n_splits runs of split_keys keys (a multiple of the key tile;
// n_splits * split_keys covers the longest visible run, counted from the tile boundary below its first key), a block a
// run, and a second kernel merges the runs.  Rows of requests that bring more are left untouched.
extern "C" int ie_attention_wide_small(const void* q, void* out, const void* kpool, const void* vpool, const int* block_table,
                                       const int* q_start, const int* ctx_before, int q_stride, int out_stride,
                                       int table_stride, int n_requests, int max_rows, int n_heads, int n_kv_heads,
                                       int page_size, int window, float scale, int chunk, int n_v_heads, int v_row,
                                       int n_splits, int split_keys, float* scratch, const float* sink,
                                       cudaStream_t stream) {
  if (n_requests <= 0) return IE_OK;
  if (max_rows <= 0 || n_splits <= 0 || n_splits > 65535) return IE_BAD_SIZE;
  if (n_splits > 1 && (split_keys <= 0 || split_keys % BN || scratch == nullptr)) return IE_BAD_SIZE;
  WideParams p;
  const int rc = wide_params(p, q, out, kpool, vpool, block_table, q_start, ctx_before, q_stride, out_stride, table_stride,
                             n_heads, n_kv_heads, page_size, window, scale, chunk, n_v_heads, v_row, sink);
  if (rc != IE_OK) return rc;
  p.tiles = (max_rows + BM - 1) / BM; p.max_rows = max_rows; p.n_splits = n_splits; p.split_keys = split_keys;
  const size_t n_parts = (size_t)n_requests * p.tiles * n_kv_heads * n_splits;
  p.part_o = scratch;
  p.part_ml = scratch != nullptr ? scratch + n_parts * BM * DV : nullptr;
  const size_t smem = wide_smem(p);
  cudaError_t e = cudaFuncSetAttribute(attention_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const dim3 grid(n_requests * p.tiles, n_kv_heads, n_splits);
  int st = launch_k(attention_wide_kernel, grid, THREADS, smem, stream, p);
  if (st != IE_OK || n_splits == 1) return st;
  return launch_k(attention_wide_merge_kernel, dim3(grid.x, grid.y, BM / MERGE_ROWS), THREADS, 0, stream, p);
}

IE_CHECK_API(attention_wide)
