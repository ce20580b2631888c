// The matrix memory of xLSTM (mLSTM) with exponential gates held stable by a running maximum.
//
// Per head, with q [dk] (already times dk^-1/2 here), k [dk], v [dv] of a token and the gate pre-activations zi, zf
// (float32, the biases added here):
//     i = cap * tanh(zi / cap)                      log input gate
//     f = logsigmoid(cap * tanh(zf / cap))          log forget gate
//     m' = max(f + m, i);   a = exp(f + m - m');   b = exp(i - m')
//     S <- a S + b k v^T;   n <- a n + b k;   m <- m'
//     o = S^T q / (max(|n . q|, exp(-m)) + 1e-6)
// S [dk, dv], n [dk] and m start at ZERO (m too: not at minus infinity) and are float32 state of the request.  The
// gates, the exponentials, the state and the quotient are float32; a step's tokens of a request run in order from the
// state that the step before left, so a whole prompt, a portion and a single decoded token take the same path and a
// cut changes nothing.
//
// Work split: a block takes one (request, head) and a chunk of value columns.  A column of S is held by P threads that
// sit side by side in a warp, each with RP = dk / P consecutive rows (P a power of two, at most MM_ROWS rows a thread);
// they add their partial sums of S^T q by shuffles.  The normaliser n obeys the very recurrence of a column of S whose
// value is always one, so the last group of P lanes of EVERY warp holds n as such a column: its sum is n . q, which
// the warp's value columns take from it by one more shuffle, and nothing crosses warps inside a tile.  Every chunk keeps
// its own copy of n and m in the state (they are the same numbers; a chunk that finishes early must not overwrite what
// another has yet to read):  state of a head = S [dk * dv], then for each chunk: n [dk], m.
// Tokens are staged a tile (up to MM_TILE) at a time in shared memory; the tile after is fetched into registers while a
// tile runs, so that no load stands in the chain of dependent steps.  Within a tile the maxima are formed one after the
// other by one thread (an addition and a comparison a token), the three exponentials of every token side by side.
//
// mlstm_finish: each head's o is divided by its root mean square over dv (eps inside the root), multiplied by a gain of
// all heads' size and by sigmoid(gate): float32, written in the activation type.
#include "common.cuh"

#define MM_ROWS 16
#define MM_TILE 16
#define MM_MAX_WARPS 4
#define MM_FETCH 12     // elements of a tile that a thread fetches ahead into registers, each of q, k and v

struct MMGeometry {
  int P, RP, cols_per_warp, chunks, chunk_cols, warps;
};

static inline bool mm_geometry(int dk, int dv, MMGeometry& g) {
  if (dk <= 0 || dv <= 0) return false;
  int p = 1;
  while (p * MM_ROWS < dk) p <<= 1;
  if (p > 16) return false;                              // a warp needs a group of lanes for n beside a value column
  g.P = p;
  g.RP = (dk + p - 1) / p;
  g.cols_per_warp = 32 / p - 1;
  const int most = MM_MAX_WARPS * g.cols_per_warp;       // value columns of a block at most
  g.chunks = (dv + most - 1) / most;
  g.chunk_cols = (dv + g.chunks - 1) / g.chunks;
  g.warps = (g.chunk_cols + g.cols_per_warp - 1) / g.cols_per_warp;
  return true;
}

extern "C" int ie_mlstm_chunks(int dk, int dv) {
  MMGeometry g;
  return mm_geometry(dk, dv, g) ? g.chunks : 0;
}

extern "C" long long ie_mlstm_state_floats(int dk, int dv) {
  const int chunks = ie_mlstm_chunks(dk, dv);
  return chunks ? (long long)dk * dv + (long long)chunks * (dk + 1) : 0;
}

// RPT > 0: every thread holds exactly RPT rows (dk = P * RPT, a multiple of 4): rows are read from shared memory in
// 16-byte pieces and nothing is guarded.  RPT = 0: any sizes, row by row with guards.
template <typename TA, typename TW, int RPT>
__global__ void __launch_bounds__(MM_MAX_WARPS * 32)
mlstm_scan_kernel(const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v, int q_stride, int k_stride,
                  int v_stride, const float* __restrict__ zi, const float* __restrict__ zf, int z_stride,
                  const TW* __restrict__ i_bias, const TW* __restrict__ f_bias, float cap, float q_scale,
                  float* __restrict__ state, long long state_stride, float* __restrict__ out, int out_stride,
                  const int* __restrict__ q_start, const int* __restrict__ slots, int dk, int dv, MMGeometry geo, int tile,
                  int write_state) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  pdl_wait();
  const int P = geo.P, RP = RPT > 0 ? RPT : geo.RP, CVB = geo.chunk_cols;
  float* sq = sm;                         // [tile][dk]
  float* sk = sq + tile * dk;             // [tile][dk]
  float* sv = sk + tile * dk;             // [tile][CVB]
  float* sg = sv + tile * CVB;            // [tile][2]: i, f; then a, b
  float* se = sg + 2 * tile;              // [tile]: exp(-m)
  float* s_m = se + tile;                 // [tile + 1]: m before the tile's first token, then after each token
  const int r_id = blockIdx.x, head = blockIdx.y, chunk = blockIdx.z;
  const int t0 = q_start[r_id], t1 = q_start[r_id + 1];
  const int slot = IE_SLOT(slots[r_id]);
  if (slot < 0 || t1 <= t0) return;
  const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int part = lane % P, group = lane / P;
  const bool is_n = group == geo.cols_per_warp;           // the warp's copy of the normaliser
  const int v0 = chunk * CVB, v_cols = min(CVB, dv - v0);
  const int col_local = warp * geo.cols_per_warp + group;
  const bool live = !is_n && col_local < v_cols;
  const int col = v0 + col_local;
  const int n_lane = geo.cols_per_warp * P;               // where the warp's n . q ends up
  float* hs = state + (size_t)slot * state_stride + (size_t)head * ((size_t)dk * dv + (size_t)geo.chunks * (dk + 1));
  float* hn = hs + (size_t)dk * dv + (size_t)chunk * (dk + 1);
  const int row0 = part * RP;
  float S[MM_ROWS];
#pragma unroll
  for (int i = 0; i < MM_ROWS; ++i) {
    const int r = row0 + i;
    const bool there = (RPT > 0 ? i < RPT : i < RP) && r < dk;
    S[i] = !there ? 0.f : (is_n ? hn[r] : (live ? hs[(size_t)r * dv + col] : 0.f));
  }
  if (tid == 0) s_m[0] = hn[dk];
  const float bi = to_f32(i_bias[head]), bf = to_f32(f_bias[head]);

  // the next tile's inputs, on their way while this tile runs; where each element of a tile lies is worked out once
  TA rq[MM_FETCH], rk[MM_FETCH], rv[MM_FETCH];
  int at_q[MM_FETCH], at_k[MM_FETCH], at_v[MM_FETCH], to_v[MM_FETCH];
#pragma unroll
  for (int j = 0; j < MM_FETCH; ++j) {
    const int idx = tid + j * nthr;
    const int tt = idx / dk, r = idx - tt * dk;
    at_q[j] = tt * q_stride + head * dk + r;
    at_k[j] = tt * k_stride + head * dk + r;
    const int tv = idx / v_cols, c = idx - tv * v_cols;
    at_v[j] = tv * v_stride + head * dv + v0 + c;
    to_v[j] = tv * CVB + c;
  }
  float rzi = 0.f, rzf = 0.f;
  auto fetch = [&](int tile0) {
    const int nt = min(tile, t1 - tile0);
    const TA* qt = q + (size_t)tile0 * q_stride;
    const TA* kt = k + (size_t)tile0 * k_stride;
    const TA* vt = v + (size_t)tile0 * v_stride;
#pragma unroll
    for (int j = 0; j < MM_FETCH; ++j) {
      const int idx = tid + j * nthr;
      if (idx < nt * dk) {
        rq[j] = qt[at_q[j]];
        rk[j] = kt[at_k[j]];
      }
      if (idx < nt * v_cols) rv[j] = vt[at_v[j]];
    }
    if (tid < nt) {
      rzi = zi[(size_t)(tile0 + tid) * z_stride + head];
      rzf = zf[(size_t)(tile0 + tid) * z_stride + head];
    }
  };
  fetch(t0);
  for (int tile0 = t0; tile0 < t1; tile0 += tile) {
    const int nt = min(tile, t1 - tile0);
    __syncthreads();                      // the tile before is used up
#pragma unroll
    for (int j = 0; j < MM_FETCH; ++j) {
      const int idx = tid + j * nthr;
      if (idx < nt * dk) {
        sq[idx] = to_f32(rq[j]) * q_scale;
        sk[idx] = to_f32(rk[j]);
      }
      if (idx < nt * v_cols) sv[to_v[j]] = to_f32(rv[j]);
    }
    if (tid < nt) {
      const float x = cap * tanhf((rzf + bf) / cap);
      sg[2 * tid] = cap * tanhf((rzi + bi) / cap);
      sg[2 * tid + 1] = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
    }
    if (tile0 + tile < t1) fetch(tile0 + tile);
    __syncthreads();
    if (tid == 0) {                       // the maxima, one after the other: additions and comparisons only
      float m = s_m[0];
      for (int tt = 0; tt < nt; ++tt) {
        m = fmaxf(sg[2 * tt + 1] + m, sg[2 * tt]);
        s_m[tt + 1] = m;
      }
    }
    __syncthreads();
    if (tid < nt) {                       // the three exponentials of every token side by side
      const float gi = sg[2 * tid], gf = sg[2 * tid + 1], m_old = s_m[tid], m_new = s_m[tid + 1];
      sg[2 * tid] = expf(gf + m_old - m_new);
      sg[2 * tid + 1] = expf(gi - m_new);
      se[tid] = expf(-m_new);
    }
    __syncthreads();
    // (vector form) the rows, the gates and the value of the token after are read while a token is worked on
    constexpr int NV = RPT > 0 ? RPT / 4 : 1;
    float4 k4[NV], q4[NV], k4n[NV], q4n[NV];
    float a_n = 0.f, b_n = 0.f, v_n = 0.f, e_n = 0.f;
    auto read_token = [&](int tt) {
      a_n = sg[2 * tt];
      b_n = sg[2 * tt + 1];
      e_n = se[tt];
      v_n = live ? sv[tt * CVB + col_local] : 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        k4n[i] = *reinterpret_cast<const float4*>(sk + tt * dk + row0 + 4 * i);
        q4n[i] = *reinterpret_cast<const float4*>(sq + tt * dk + row0 + 4 * i);
      }
    };
    if (RPT > 0) read_token(0);
    for (int tt = 0; tt < nt; ++tt) {
      float a, b, x, e_here;
      const float* qr = sq + tt * dk + row0;
      const float* kr = sk + tt * dk + row0;
      float acc0 = 0.f, acc1 = 0.f;
      if (RPT > 0) {
        a = a_n; b = b_n; e_here = e_n;
        x = is_n ? b : b * v_n;            // one for the normaliser's column, nothing for a column beyond the head
#pragma unroll
        for (int i = 0; i < NV; ++i) { k4[i] = k4n[i]; q4[i] = q4n[i]; }
        if (tt + 1 < nt) read_token(tt + 1);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          S[4 * i] = fmaf(a, S[4 * i], k4[i].x * x);
          S[4 * i + 1] = fmaf(a, S[4 * i + 1], k4[i].y * x);
          S[4 * i + 2] = fmaf(a, S[4 * i + 2], k4[i].z * x);
          S[4 * i + 3] = fmaf(a, S[4 * i + 3], k4[i].w * x);
          acc0 = fmaf(S[4 * i], q4[i].x, acc0);
          acc1 = fmaf(S[4 * i + 1], q4[i].y, acc1);
          acc0 = fmaf(S[4 * i + 2], q4[i].z, acc0);
          acc1 = fmaf(S[4 * i + 3], q4[i].w, acc1);
        }
      } else {
        a = sg[2 * tt]; b = sg[2 * tt + 1]; e_here = se[tt];
        x = is_n ? b : (live ? b * sv[tt * CVB + col_local] : 0.f);
#pragma unroll
        for (int i = 0; i < MM_ROWS; ++i) {
          if (i < RP && row0 + i < dk) {
            S[i] = fmaf(a, S[i], kr[i] * x);
            if (i & 1) acc1 = fmaf(S[i], qr[i], acc1); else acc0 = fmaf(S[i], qr[i], acc0);
          }
        }
      }
      float acc = acc0 + acc1;
      for (int o = 1; o < P; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const float nq = __shfl_sync(0xffffffffu, acc, n_lane);
      if (live && part == 0)
        out[(size_t)(tile0 + tt) * out_stride + head * dv + col] = acc / (fmaxf(fabsf(nq), e_here) + 1e-6f);
    }
    if (tid == 0) s_m[0] = s_m[nt];       // (read again only after the next barrier)
  }
  if (!write_state) return;
#pragma unroll
  for (int i = 0; i < MM_ROWS; ++i) {
    const int r = row0 + i;
    if ((RPT > 0 ? i < RPT : i < RP) && r < dk) {
      if (live) hs[(size_t)r * dv + col] = S[i];
      if (is_n && warp == 0) hn[r] = S[i];
    }
  }
  if (tid == 0) hn[dk] = s_m[0];
}

extern "C" int ie_mlstm_scan(const void* q, const void* k, const void* v, int q_stride, int k_stride, int v_stride,
                             const float* zi, const float* zf, int z_stride, const void* i_bias, const void* f_bias,
                             int w_dtype, float cap, float q_scale, float* state, long long state_stride, float* out,
                             int out_stride, const int* q_start, const int* slots, int n_requests, int heads, int dk,
                             int dv, int write_state, int act_dtype, cudaStream_t stream) {
  if (n_requests <= 0) return IE_OK;
  if (heads <= 0 || heads > 65535 || !(cap > 0.f)) return IE_BAD_SIZE;
  MMGeometry g;
  if (!mm_geometry(dk, dv, g) || g.chunks > 65535) return IE_BAD_SIZE;
  const int threads = g.warps * 32;
  // tokens of a tile: what a thread can fetch ahead in MM_FETCH elements each of q, k and v
  int tile = (MM_FETCH * threads) / (dk > g.chunk_cols ? dk : g.chunk_cols);
  if (tile > MM_TILE) tile = MM_TILE;
  if (tile > threads) tile = threads;
  if (tile < 1) return IE_BAD_SIZE;
  const size_t smem = sizeof(float) * ((size_t)2 * tile * dk + (size_t)tile * g.chunk_cols + 4 * tile + 1);
  if (smem > 48 * 1024) return IE_BAD_SIZE;
  dim3 grid(n_requests, heads, g.chunks);
  // rows in 16-byte pieces when every thread holds the same multiple of four rows
  const int rpt = (dk == g.P * g.RP && (g.RP & 3) == 0) ? g.RP : 0;
#define MM_LAUNCH(TA, TW, R)                                                                                          \
  return launch_k(mlstm_scan_kernel<TA, TW, R>, grid, threads, smem, stream, (const TA*)q, (const TA*)k, (const TA*)v, \
                  q_stride, k_stride, v_stride, zi, zf, z_stride, (const TW*)i_bias, (const TW*)f_bias, cap, q_scale,  \
                  state, state_stride, out, out_stride, q_start, slots, dk, dv, g, tile, write_state)
#define MM_GO(TA, TW)               \
  {                                 \
    if (rpt == 16) MM_LAUNCH(TA, TW, 16); \
    if (rpt == 12) MM_LAUNCH(TA, TW, 12); \
    if (rpt == 8) MM_LAUNCH(TA, TW, 8);   \
    if (rpt == 4) MM_LAUNCH(TA, TW, 4);   \
    MM_LAUNCH(TA, TW, 0);           \
  }
  if (act_dtype == IE_F32 && w_dtype == IE_F32) MM_GO(float, float);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) MM_GO(float, bf16);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) MM_GO(bf16, float);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) MM_GO(bf16, bf16);
#undef MM_GO
#undef MM_LAUNCH
  return IE_BAD_DTYPE;
}

// a warp a (token, head)
template <typename TA, typename TW>
__global__ void mlstm_finish_kernel(const float* __restrict__ o, int o_stride, const TW* __restrict__ gain,
                                    const TA* __restrict__ gate, int gate_stride, TA* __restrict__ out, int out_stride,
                                    int n, int heads, int dv, float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n * heads) return;
  const int t = (int)(w / heads), h = (int)(w - (long long)t * heads);
  const float* row = o + (size_t)t * o_stride + h * dv;
  if (sizeof(TA) == 2 && sizeof(TW) == 2 && (dv & 63) == 0 && ((o_stride | gate_stride | out_stride) & 1) == 0) {
    // pairs of neighbouring coordinates: 8-byte loads of o, 4-byte ones of gain, gate and result
    float ss = 0.f;
    for (int d = 2 * lane; d < dv; d += 64) {
      const float2 v = *reinterpret_cast<const float2*>(row + d);
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, ss));
    }
    ss = warp_sum(ss);
    const float r = sqrtf(ss / (float)dv + eps);
    for (int d = 2 * lane; d < dv; d += 64) {
      const int c = h * dv + d;
      const float2 v = *reinterpret_cast<const float2*>(row + d);
      const float2 gn = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gain + c));
      const float2 z = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + (size_t)t * gate_stride + c));
      *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * out_stride + c) =
          __floats2bfloat162_rn(v.x / r * gn.x / (1.f + expf(-z.x)), v.y / r * gn.y / (1.f + expf(-z.y)));
    }
    return;
  }
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss = fmaf(row[d], row[d], ss);
  ss = warp_sum(ss);
  const float r = sqrtf(ss / (float)dv + eps);
  for (int d = lane; d < dv; d += 32) {
    const int c = h * dv + d;
    const float z = to_f32(gate[(size_t)t * gate_stride + c]);
    out[(size_t)t * out_stride + c] = from_f32<TA>(row[d] / r * to_f32(gain[c]) / (1.f + expf(-z)));
  }
}

extern "C" int ie_mlstm_finish(const float* o, int o_stride, const void* gain, int w_dtype, const void* gate,
                               int gate_stride, void* out, int out_stride, int n, int heads, int dv, float eps,
                               int act_dtype, cudaStream_t stream) {
  if (n <= 0) return IE_OK;
  if (heads <= 0 || dv <= 0) return IE_BAD_SIZE;
  const unsigned blocks = (unsigned)(((long long)n * heads + 7) / 8);
#define MF_GO(TA, TW)                                                                                               \
  return launch_k(mlstm_finish_kernel<TA, TW>, blocks, 256, 0, stream, o, o_stride, (const TW*)gain, (const TA*)gate, \
                  gate_stride, (TA*)out, out_stride, n, heads, dv, eps)
  if (act_dtype == IE_F32 && w_dtype == IE_F32) MF_GO(float, float);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) MF_GO(float, bf16);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) MF_GO(bf16, float);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) MF_GO(bf16, bf16);
#undef MF_GO
  return IE_BAD_DTYPE;
}

IE_CHECK_API(matrix_memory)
