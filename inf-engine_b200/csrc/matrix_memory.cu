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
// Work split: a block takes one (request, head) and a chunk of CV value columns; a thread holds, for one column, the
// rows p, p + P, p + 2 P, ... of S (at most MM_ROWS of them) and the same rows of n; the P threads of a column sit side
// by side in a warp and add their partial sums by shuffles.  Every chunk keeps its own copy of n and m in the state
// (they are the same numbers; a chunk that finishes early must not overwrite what another has yet to read):
//     state of a head = S [dk * dv], then for each chunk: n [dk], m.
// Tokens are staged MM_TILE at a time in shared memory.
//
// mlstm_finish: each head's o is divided by its root mean square over dv (eps inside the root), multiplied by a gain of
// all heads' size and by sigmoid(gate): float32, written in the activation type.
#include "common.cuh"

#define MM_ROWS 16
#define MM_TILE 16
#define MM_THREADS 256

static inline int mm_parts(int dk) {
  int p = 1;
  while (p * MM_ROWS < dk) p <<= 1;
  return p;
}
static inline int mm_chunk_cols(int dk, int dv) {
  const int cv = MM_THREADS / mm_parts(dk);
  return dv < cv ? dv : cv;
}

extern "C" int ie_mlstm_chunks(int dk, int dv) {
  if (dk <= 0 || dv <= 0 || mm_parts(dk) > 32) return 0;
  const int cv = mm_chunk_cols(dk, dv);
  return (dv + cv - 1) / cv;
}

extern "C" long long ie_mlstm_state_floats(int dk, int dv) {
  const int chunks = ie_mlstm_chunks(dk, dv);
  return chunks ? (long long)dk * dv + (long long)chunks * (dk + 1) : 0;
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(MM_THREADS)
mlstm_scan_kernel(const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v, int q_stride, int k_stride,
                  int v_stride, const float* __restrict__ zi, const float* __restrict__ zf, int z_stride,
                  const TW* __restrict__ i_bias, const TW* __restrict__ f_bias, float cap, float q_scale,
                  float* __restrict__ state, long long state_stride, float* __restrict__ out, int out_stride,
                  const int* __restrict__ q_start, const int* __restrict__ slots, int heads, int dk, int dv, int P, int CV,
                  int write_state) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  float* sq = sm;                         // [MM_TILE][dk]
  float* sk = sq + MM_TILE * dk;          // [MM_TILE][dk]
  float* sv = sk + MM_TILE * dk;          // [MM_TILE][CV]
  float* sg = sv + MM_TILE * CV;          // [MM_TILE][2]: i, f
  const int r_id = blockIdx.x, head = blockIdx.y, chunk = blockIdx.z;
  const int t0 = q_start[r_id], t1 = q_start[r_id + 1];
  const int slot = IE_SLOT(slots[r_id]);
  if (slot < 0 || t1 <= t0) return;
  const int part = threadIdx.x % P, col_local = threadIdx.x / P;
  const int col = chunk * CV + col_local;
  const bool live = col_local < CV && col < dv;
  const int n_chunks = (dv + CV - 1) / CV;
  float* hs = state + (size_t)slot * state_stride + (size_t)head * ((size_t)dk * dv + (size_t)n_chunks * (dk + 1));
  float* hn = hs + (size_t)dk * dv + (size_t)chunk * (dk + 1);
  float S[MM_ROWS], nn[MM_ROWS];
#pragma unroll
  for (int i = 0; i < MM_ROWS; ++i) {
    const int r = part + P * i;
    S[i] = (live && r < dk) ? hs[(size_t)r * dv + col] : 0.f;
    nn[i] = r < dk ? hn[r] : 0.f;
  }
  float m = hn[dk];
  const float bi = to_f32(i_bias[head]), bf = to_f32(f_bias[head]);
  for (int tile0 = t0; tile0 < t1; tile0 += MM_TILE) {
    const int nt = min(MM_TILE, t1 - tile0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * dk; idx += blockDim.x) {
      const int tt = idx / dk, r = idx - tt * dk;
      sq[idx] = to_f32(q[(size_t)(tile0 + tt) * q_stride + head * dk + r]) * q_scale;
      sk[idx] = to_f32(k[(size_t)(tile0 + tt) * k_stride + head * dk + r]);
    }
    for (int idx = threadIdx.x; idx < nt * CV; idx += blockDim.x) {
      const int tt = idx / CV, c = idx - tt * CV;
      sv[idx] = chunk * CV + c < dv ? to_f32(v[(size_t)(tile0 + tt) * v_stride + head * dv + chunk * CV + c]) : 0.f;
    }
    for (int tt = threadIdx.x; tt < nt; tt += blockDim.x) {
      const float ai = zi[(size_t)(tile0 + tt) * z_stride + head] + bi;
      const float af = zf[(size_t)(tile0 + tt) * z_stride + head] + bf;
      const float x = cap * tanhf(af / cap);
      sg[2 * tt] = cap * tanhf(ai / cap);
      sg[2 * tt + 1] = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float gi = sg[2 * tt], gf = sg[2 * tt + 1];
      const float m_new = fmaxf(gf + m, gi);
      const float a = expf(gf + m - m_new), b = expf(gi - m_new);
      m = m_new;
      const float* qr = sq + tt * dk;
      const float* kr = sk + tt * dk;
      const float bv = b * sv[tt * CV + (col_local < CV ? col_local : 0)];
      float acc = 0.f, nq = 0.f;
#pragma unroll
      for (int i = 0; i < MM_ROWS; ++i) {
        const int r = part + P * i;
        if (r < dk) {
          const float kv = kr[r], qv = qr[r];
          S[i] = fmaf(a, S[i], kv * bv);
          nn[i] = fmaf(a, nn[i], b * kv);
          acc = fmaf(S[i], qv, acc);
          nq = fmaf(nn[i], qv, nq);
        }
      }
      for (int o = 1; o < P; o <<= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
        nq += __shfl_xor_sync(0xffffffffu, nq, o);
      }
      if (live && part == 0)
        out[(size_t)(tile0 + tt) * out_stride + head * dv + col] = acc / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
    }
  }
  if (!write_state) return;
#pragma unroll
  for (int i = 0; i < MM_ROWS; ++i) {
    const int r = part + P * i;
    if (r < dk) {
      if (live) hs[(size_t)r * dv + col] = S[i];
      if (col_local == 0) hn[r] = nn[i];
    }
  }
  if (threadIdx.x == 0) hn[dk] = m;
}

extern "C" int ie_mlstm_scan(const void* q, const void* k, const void* v, int q_stride, int k_stride, int v_stride,
                             const float* zi, const float* zf, int z_stride, const void* i_bias, const void* f_bias,
                             int w_dtype, float cap, float q_scale, float* state, long long state_stride, float* out,
                             int out_stride, const int* q_start, const int* slots, int n_requests, int heads, int dk,
                             int dv, int write_state, int act_dtype, cudaStream_t stream) {
  if (n_requests <= 0) return IE_OK;
  if (heads <= 0 || heads > 65535 || dk <= 0 || dv <= 0 || !(cap > 0.f)) return IE_BAD_SIZE;
  const int P = mm_parts(dk);
  if (P > 32) return IE_BAD_SIZE;
  const int CV = mm_chunk_cols(dk, dv);
  const int chunks = (dv + CV - 1) / CV;
  if (chunks > 65535) return IE_BAD_SIZE;
  const size_t smem = sizeof(float) * ((size_t)2 * MM_TILE * dk + (size_t)MM_TILE * CV + 2 * MM_TILE);
  if (smem > 48 * 1024) return IE_BAD_SIZE;
  dim3 grid(n_requests, heads, chunks);
  // whole warps, so that the shuffles of a column's threads always find their partners
  const int threads = ((CV * P + 31) / 32) * 32;
#define MM_GO(TA, TW)                                                                                              \
  return launch_k(mlstm_scan_kernel<TA, TW>, grid, threads, smem, stream, (const TA*)q, (const TA*)k, (const TA*)v, \
                  q_stride, k_stride, v_stride, zi, zf, z_stride, (const TW*)i_bias, (const TW*)f_bias, cap, q_scale, \
                  state, state_stride, out, out_stride, q_start, slots, heads, dk, dv, P, CV, write_state)
  if (act_dtype == IE_F32 && w_dtype == IE_F32) MM_GO(float, float);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) MM_GO(float, bf16);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) MM_GO(bf16, float);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) MM_GO(bf16, bf16);
#undef MM_GO
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
