// Kernels for layers that put their norm on a sublayer's output and for mixers that carry a state along the
// sequence: a cast of the float32 residual rows to the activation type, an RMS norm of a sublayer's output added
// into the residual, a short causal convolution per channel whose last inputs are state, the scan of a real-gated
// linear recurrent unit, and an RMS norm over whole query and key rows fused with the rotation of neighbouring
// pairs and the write of keys and values into cache pages.  Statistics, angles, gates, decays and states are
// float32 whatever the activation type is.
#include "common.cuh"

// ------------------------------------------------------------------ residual rows in the activation type
template <typename TA>
__global__ void cast_rows_kernel(const float* __restrict__ x, TA* __restrict__ out, long long n) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f32<TA>(x[i]);
}

extern "C" int ie_cast_rows(const float* x, void* out, int out_dtype, int n_rows, int d, cudaStream_t stream) {
  const long long n = (long long)n_rows * d;
  if (n <= 0) return IE_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (out_dtype == IE_BF16) return launch_k(cast_rows_kernel<bf16>, blocks, 256, 0, stream, x, (bf16*)out, n);
  if (out_dtype == IE_F32) return launch_k(cast_rows_kernel<float>, blocks, 256, 0, stream, x, (float*)out, n);
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ norm of a sublayer's output into the residual
// residual[row] += y[row] / sqrt(mean(y[row]^2) + eps) * gain;  next_in[row] = residual[row] in the activation type
// (the input of the sublayer that follows, if asked for).  One block per row, y staged in shared memory.
template <typename TY, typename TW, typename TA>
__global__ void outnorm_accumulate_kernel(float* __restrict__ residual, const TY* __restrict__ y, int y_stride,
                                          const TW* __restrict__ gain, TA* __restrict__ next_in, int d, float eps) {
  extern __shared__ float ys[];
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const TY* yr = y + (size_t)row * y_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = to_f32(yr[i]);
    ys[i] = v;
    ss += v * v;
  }
  const float rms = sqrtf(block_sum(ss, red) / (float)d + eps);
  float* res = residual + (size_t)row * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float x = res[i] + (ys[i] / rms) * to_f32(gain[i]);
    res[i] = x;
    if (next_in != nullptr) next_in[(size_t)row * d + i] = from_f32<TA>(x);
  }
}

template <typename TY, typename TW>
static int launch_outnorm(float* residual, const void* y, int y_stride, const void* gain, void* next_in, int next_dtype,
                          int n_rows, int d, float eps, cudaStream_t stream) {
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return IE_BAD_SIZE;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  if (next_in == nullptr || next_dtype == IE_BF16) {
    if (smem > 47 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(outnorm_accumulate_kernel<TY, TW, bf16>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return launch_k(outnorm_accumulate_kernel<TY, TW, bf16>, n_rows, threads, smem, stream, residual, (const TY*)y,
                    y_stride, (const TW*)gain, (bf16*)next_in, d, eps);
  }
  if (next_dtype != IE_F32) return IE_BAD_DTYPE;
  if (smem > 47 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(outnorm_accumulate_kernel<TY, TW, float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_k(outnorm_accumulate_kernel<TY, TW, float>, n_rows, threads, smem, stream, residual, (const TY*)y,
                  y_stride, (const TW*)gain, (float*)next_in, d, eps);
}

extern "C" int ie_outnorm_accumulate(float* residual, const void* y, int y_dtype, int y_stride, const void* gain,
                                     int gain_dtype, void* next_in, int next_dtype, int n_rows, int d, float eps,
                                     cudaStream_t stream) {
  if (n_rows <= 0) return IE_OK;
  if (y_dtype == IE_F32 && gain_dtype == IE_F32)
    return launch_outnorm<float, float>(residual, y, y_stride, gain, next_in, next_dtype, n_rows, d, eps, stream);
  if (y_dtype == IE_F32 && gain_dtype == IE_BF16)
    return launch_outnorm<float, bf16>(residual, y, y_stride, gain, next_in, next_dtype, n_rows, d, eps, stream);
  if (y_dtype == IE_BF16 && gain_dtype == IE_F32)
    return launch_outnorm<bf16, float>(residual, y, y_stride, gain, next_in, next_dtype, n_rows, d, eps, stream);
  if (y_dtype == IE_BF16 && gain_dtype == IE_BF16)
    return launch_outnorm<bf16, bf16>(residual, y, y_stride, gain, next_in, next_dtype, n_rows, d, eps, stream);
  return IE_BAD_DTYPE;
}

// The same, followed by the norm that the residual meets next: normed[row] = x / sqrt(mean(x^2) + eps2) * gain2 with x
// the new residual row (kept in shared memory between the two sums), in the activation type.
template <typename TY, typename TW, typename TW2, typename TA>
__global__ void outnorm_accumulate_norm_kernel(float* __restrict__ residual, const TY* __restrict__ y, int y_stride,
                                               const TW* __restrict__ gain, float eps, const TW2* __restrict__ gain2,
                                               float eps2, TA* __restrict__ normed, int d) {
  extern __shared__ float ys[];
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const TY* yr = y + (size_t)row * y_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = to_f32(yr[i]);
    ys[i] = v;
    ss += v * v;
  }
  const float rms = sqrtf(block_sum(ss, red) / (float)d + eps);
  float* res = residual + (size_t)row * d;
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float x = res[i] + (ys[i] / rms) * to_f32(gain[i]);
    res[i] = x;
    ys[i] = x;
    ss2 += x * x;
  }
  const float rms2 = sqrtf(block_sum(ss2, red) / (float)d + eps2);
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    normed[(size_t)row * d + i] = from_f32<TA>(ys[i] / rms2 * to_f32(gain2[i]));
}

extern "C" int ie_outnorm_accumulate_norm(float* residual, const void* y, int y_dtype, int y_stride, const void* gain,
                                          int gain_dtype, float eps, const void* gain2, int gain2_dtype, float eps2,
                                          void* normed, int normed_dtype, int n_rows, int d, cudaStream_t stream) {
  if (n_rows <= 0) return IE_OK;
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return IE_BAD_SIZE;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
#define ON_GO(TY, TW, TW2, TA)                                                                                          \
  {                                                                                                                     \
    if (smem > 47 * 1024) {                                                                                             \
      cudaError_t e = cudaFuncSetAttribute(outnorm_accumulate_norm_kernel<TY, TW, TW2, TA>,                             \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                    \
      if (e != cudaSuccess) return (int)e;                                                                              \
    }                                                                                                                   \
    return launch_k(outnorm_accumulate_norm_kernel<TY, TW, TW2, TA>, n_rows, threads, smem, stream, residual,           \
                    (const TY*)y, y_stride, (const TW*)gain, eps, (const TW2*)gain2, eps2, (TA*)normed, d);              \
  }
#define ON_GAINS(TY, TA)                                                          \
  {                                                                               \
    if (gain_dtype == IE_F32 && gain2_dtype == IE_F32) ON_GO(TY, float, float, TA); \
    if (gain_dtype == IE_BF16 && gain2_dtype == IE_BF16) ON_GO(TY, bf16, bf16, TA); \
    return IE_BAD_DTYPE;                                                          \
  }
  if (y_dtype == IE_F32 && normed_dtype == IE_F32) ON_GAINS(float, float);
  if (y_dtype == IE_F32 && normed_dtype == IE_BF16) ON_GAINS(float, bf16);
  if (y_dtype == IE_BF16 && normed_dtype == IE_BF16) ON_GAINS(bf16, bf16);
  if (y_dtype == IE_BF16 && normed_dtype == IE_F32) ON_GAINS(bf16, float);
#undef ON_GAINS
#undef ON_GO
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ short causal convolution with state
// out[t, c] = act(bias[c] + sum_j w[c, j] * x[t - (taps - 1 - j), c]): the last column of w multiplies the current
// token's input.  Inputs before the first token of the step come from the request's state, [taps - 1, channels] in
// the activation type (the last inputs of the sequence so far, oldest first; zero when the sequence starts), and the
// state is then moved on by the step's tokens.  A block owns 32 channels of one chunk of 64 tokens of one request: its
// 8 rows of threads take the chunk's tokens in turn.  Only a request's first chunk reads the old state, and that
// block, when all its rows have read what they need of it, writes the new one (from the request's last tokens of the
// step, which no kernel writes meanwhile).  So any cut of a sequence into steps gives the same outputs.
#define CONV_CH 32
#define CONV_TL 8
#define CONV_CHUNK 64
#define CONV_MAX_TAPS 16

template <typename TA, typename TW>
__global__ void __launch_bounds__(CONV_CH* CONV_TL)
causal_conv_kernel(const TA* __restrict__ x, int x_stride, const TW* __restrict__ w, const TW* __restrict__ bias,
                   TA* __restrict__ state, long long state_slot_stride, TA* __restrict__ out, int out_stride,
                   const int* __restrict__ q_start, const int* __restrict__ slots, int channels, int taps,
                   int activation, int write_state) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * CONV_CH + threadIdx.x;
  const int tl = threadIdx.y;
  const int req = blockIdx.y;
  const int q0 = q_start[req], q1 = q_start[req + 1];
  const int t_lo = q0 + blockIdx.z * CONV_CHUNK, t_hi = min(q1, t_lo + CONV_CHUNK);
  if (t_lo >= q1 && blockIdx.z > 0) return;                  // a shorter request than the step's longest
  const int slot = IE_SLOT(slots[req]);
  const bool live = c < channels;
  TA* st = (slot >= 0 && live) ? state + (size_t)slot * state_slot_stride + c : nullptr;   // element i at st[i * channels]
  float wv[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) wv[j] = (live && j < taps) ? to_f32(w[(size_t)c * taps + j]) : 0.f;
  const float b = (live && bias != nullptr) ? to_f32(bias[c]) : 0.f;
  if (live) {
    for (int t = t_lo + tl; t < t_hi; t += CONV_TL) {
      float acc = b;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        if (j < taps) {
          const int src = t - (taps - 1 - j);
          float xv = 0.f;
          if (src >= q0) xv = to_f32(x[(size_t)src * x_stride + c]);
          else if (st != nullptr) xv = to_f32(st[(size_t)(taps - 1 - (q0 - src)) * channels]);
          acc = fmaf(wv[j], xv, acc);
        }
      }
      if (activation == 1) acc = acc / (1.f + expf(-acc));
      out[(size_t)t * out_stride + c] = from_f32<TA>(acc);
    }
  }
  if (blockIdx.z > 0) return;
  __syncthreads();
  if (write_state && st != nullptr && tl == 0) {
    const int n = q1 - q0, keep = taps - 1;
    float nv[CONV_MAX_TAPS];
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i) {
      nv[i] = 0.f;
      if (i < keep) {
        const int src = q1 - keep + i;             // the token that ends up at place i
        nv[i] = src >= q0 ? to_f32(x[(size_t)src * x_stride + c]) : to_f32(st[(size_t)(i + n) * channels]);
      }
    }
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i)
      if (i < keep) st[(size_t)i * channels] = from_f32<TA>(nv[i]);
  }
}

extern "C" int ie_causal_conv(const void* x, int x_stride, const void* w, const void* bias, int w_dtype, void* state,
                              long long state_slot_stride, void* out, int out_stride, const int* q_start,
                              const int* slots, int n_requests, int channels, int taps, int activation,
                              int write_state, int act_dtype, int max_q_len, cudaStream_t stream) {
  if (n_requests <= 0 || channels <= 0) return IE_OK;
  if (taps < 1 || taps > CONV_MAX_TAPS || max_q_len < 1) return IE_BAD_SIZE;
  const int chunks = (max_q_len + CONV_CHUNK - 1) / CONV_CHUNK;       // of the step's longest request
  if (chunks > 65535) return IE_BAD_SIZE;
  dim3 grid((channels + CONV_CH - 1) / CONV_CH, n_requests, chunks), block(CONV_CH, CONV_TL);
#define CONV_GO(TA, TW)                                                                                          \
  return launch_k(causal_conv_kernel<TA, TW>, grid, block, 0, stream, (const TA*)x, x_stride, (const TW*)w,      \
                  (const TW*)bias, (TA*)state, state_slot_stride, (TA*)out, out_stride, q_start, slots, channels, \
                  taps, activation, write_state)
  if (act_dtype == IE_F32 && w_dtype == IE_F32) CONV_GO(float, float);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) CONV_GO(float, bf16);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) CONV_GO(bf16, float);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) CONV_GO(bf16, bf16);
#undef CONV_GO
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ real-gated linear recurrent unit
// Per channel, token after token, from the request's float32 state S (zero when the sequence starts):
//     r = sigmoid(r_pre + r_bias),  i = sigmoid(i_pre + i_bias)             (r_pre, i_pre: float32 gate products)
//     log a = -decay_scale * r * softplus(lam),  a = exp(log a)
//     S <- a S + sqrt(1 - a^2) (i * u);    out = out_scale * S * gelu_tanh(y_pre)
// 1 - a^2 is formed as -expm1(2 log a), which keeps its digits when a is close to one; and while a is above one
// half the state is moved by S += (a - 1) S + input with a - 1 = expm1(log a): a float32 a = 1 - 2.5e-6 is off by up
// to a hundredth of its distance from one, which over a thousand tokens shows in the fifth digit of S.  A thread owns a channel
// of a request and walks the step's tokens in order; the loads of a token do not depend on S, so several
// tokens' loads are in flight while the chain runs.
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// S <- exp(log_a) S + in, log_a <= 0
__device__ __forceinline__ float lru_step(float S, float log_a, float in) {
  if (log_a > -0.6931472f) return S + fmaf(expm1f(log_a), S, in);
  return fmaf(expf(log_a), S, in);
}

#define LRU_UNROLL 4
template <typename TA, typename TW>
__global__ void __launch_bounds__(128)
linear_recurrence_kernel(const TA* __restrict__ u, int u_stride, const TA* __restrict__ y_pre, int y_stride,
                         const float* __restrict__ r_pre, const float* __restrict__ i_pre, int g_stride,
                         const TW* __restrict__ r_bias, const TW* __restrict__ i_bias, const TW* __restrict__ lam,
                         float* __restrict__ state, TA* __restrict__ out, int out_stride,
                         const int* __restrict__ q_start, const int* __restrict__ slots, int width,
                         float decay_scale, float out_scale, int write_state) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int req = blockIdx.y;
  if (c >= width) return;
  const int q0 = q_start[req], q1 = q_start[req + 1];
  const int slot = IE_SLOT(slots[req]);
  if (slot < 0) {
    for (int t = q0; t < q1; ++t) out[(size_t)t * out_stride + c] = from_f32<TA>(0.f);
    return;
  }
  const float rb = to_f32(r_bias[c]), ib = to_f32(i_bias[c]);
  const float rate = -decay_scale * softplus_f(to_f32(lam[c]));
  float S = state[(size_t)slot * width + c];
  int t = q0;
  for (; t + LRU_UNROLL <= q1; t += LRU_UNROLL) {
    float rp[LRU_UNROLL], ip[LRU_UNROLL], uu[LRU_UNROLL], yy[LRU_UNROLL];
#pragma unroll
    for (int k = 0; k < LRU_UNROLL; ++k) {
      rp[k] = r_pre[(size_t)(t + k) * g_stride + c];
      ip[k] = i_pre[(size_t)(t + k) * g_stride + c];
      uu[k] = to_f32(u[(size_t)(t + k) * u_stride + c]);
      yy[k] = to_f32(y_pre[(size_t)(t + k) * y_stride + c]);
    }
#pragma unroll
    for (int k = 0; k < LRU_UNROLL; ++k) {
      const float log_a = rate * sigmoid_f(rp[k] + rb);
      const float in = sqrtf(-expm1f(2.f * log_a)) * (sigmoid_f(ip[k] + ib) * uu[k]);
      S = lru_step(S, log_a, in);
      out[(size_t)(t + k) * out_stride + c] = from_f32<TA>(out_scale * S * gelu_tanh_f(yy[k]));
    }
  }
  for (; t < q1; ++t) {
    const float log_a = rate * sigmoid_f(r_pre[(size_t)t * g_stride + c] + rb);
    const float in = sqrtf(-expm1f(2.f * log_a)) *
                     (sigmoid_f(i_pre[(size_t)t * g_stride + c] + ib) * to_f32(u[(size_t)t * u_stride + c]));
    S = lru_step(S, log_a, in);
    out[(size_t)t * out_stride + c] =
        from_f32<TA>(out_scale * S * gelu_tanh_f(to_f32(y_pre[(size_t)t * y_stride + c])));
  }
  if (write_state) state[(size_t)slot * width + c] = S;
}

extern "C" int ie_linear_recurrence(const void* u, int u_stride, const void* y_pre, int y_stride, const float* r_pre,
                                    const float* i_pre, int g_stride, const void* r_bias, const void* i_bias,
                                    const void* lam, int w_dtype, float* state, void* out, int out_stride,
                                    const int* q_start, const int* slots, int n_requests, int width,
                                    float decay_scale, float out_scale, int write_state, int act_dtype,
                                    cudaStream_t stream) {
  if (n_requests <= 0 || width <= 0) return IE_OK;
  dim3 grid((width + 127) / 128, n_requests);
#define LRU_GO(TA, TW)                                                                                             \
  return launch_k(linear_recurrence_kernel<TA, TW>, grid, 128, 0, stream, (const TA*)u, u_stride, (const TA*)y_pre, \
                  y_stride, r_pre, i_pre, g_stride, (const TW*)r_bias, (const TW*)i_bias, (const TW*)lam, state,    \
                  (TA*)out, out_stride, q_start, slots, width, decay_scale, out_scale, write_state)
  if (act_dtype == IE_F32 && w_dtype == IE_F32) LRU_GO(float, float);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) LRU_GO(float, bf16);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) LRU_GO(bf16, float);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) LRU_GO(bf16, bf16);
#undef LRU_GO
  return IE_BAD_DTYPE;
}

// ------------------------------------------------- whole-row norm of q and k, pair rotation, cache write
// For every token: q <- q + q_bias, divided by the root mean square of the WHOLE row (all heads together; eps inside
// the root) and multiplied by a gain of the row's size; the same for k; v <- v + v_bias.  Then, in every head of q
// and k, the first rot_dims dimensions turn in neighbouring pairs: (a, b) at dimensions (2i, 2i + 1) becomes
// (a cos - b sin, b cos + a sin) of the angle position * inv_freq[i] (float64 frequencies).  q is
// written back in place; k and v go to the token's place in the cache pages (and nowhere else).  A null gain or
// bias leaves that step out.  One block per token; the normed rows are staged in shared memory.
template <typename TA, typename TW>
__global__ void rownorm_rotate_write_kernel(TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v,
                                            int q_stride, int k_stride, int v_stride, const TW* __restrict__ q_bias,
                                            const TW* __restrict__ k_bias, const TW* __restrict__ v_bias,
                                            const TW* __restrict__ q_gain, const TW* __restrict__ k_gain, float eps,
                                            const double* __restrict__ inv_freq, int rot_dims,
                                            const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                            TA* __restrict__ kpool, TA* __restrict__ vpool, int n_heads,
                                            int n_kv_heads, int hd, int hd_v, int page_size) {
  extern __shared__ float rows[];
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int qw = n_heads * hd, kw = n_kv_heads * hd, vw = n_kv_heads * hd_v;
  float* qs = rows;
  float* ks = rows + qw;
  TA* qr = q + (size_t)n * q_stride;
  const TA* kr = k + (size_t)n * k_stride;
  const TA* vr = v + (size_t)n * v_stride;
  float ssq = 0.f, ssk = 0.f;
  for (int i = threadIdx.x; i < qw; i += blockDim.x) {
    const float x = to_f32(qr[i]) + (q_bias ? to_f32(q_bias[i]) : 0.f);
    qs[i] = x;
    ssq += x * x;
  }
  for (int i = threadIdx.x; i < kw; i += blockDim.x) {
    const float x = to_f32(kr[i]) + (k_bias ? to_f32(k_bias[i]) : 0.f);
    ks[i] = x;
    ssk += x * x;
  }
  const float q_rms = q_gain ? sqrtf(block_sum(ssq, red) / (float)qw + eps) : 1.f;
  const float k_rms = k_gain ? sqrtf(block_sum(ssk, red) / (float)kw + eps) : 1.f;
  __syncthreads();
  if (q_gain)
    for (int i = threadIdx.x; i < qw; i += blockDim.x) qs[i] = qs[i] / q_rms * to_f32(q_gain[i]);
  if (k_gain)
    for (int i = threadIdx.x; i < kw; i += blockDim.x) ks[i] = ks[i] / k_rms * to_f32(k_gain[i]);
  __syncthreads();
  const float pos = (float)positions[n];
  const int slot = slot_mapping ? IE_SLOT(slot_mapping[n]) : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  for (int i = threadIdx.x; i < qw + kw; i += blockDim.x) {
    const bool is_q = i < qw;
    const int e = is_q ? i : i - qw;
    const float* src = is_q ? qs : ks;
    const int h = e / hd, le = e - h * hd;
    float val = src[e];
    if (le < rot_dims) {
      const int pair = le >> 1;
      float sn, cs;
#ifdef IE_ANGLE_F32
      sincosf(pos * (float)inv_freq[pair], &sn, &cs);
#else
      // frequency times position is formed and brought into one turn in double, then the sine and cosine are float32:
      // a float32 product at position 100,000 would be off by a thousandth of a radian before any sine is taken, and
      // a frequency rounded to float32 puts a key 1,000 positions back off by 3e-5 of a radian
      const double turns = (double)pos * inv_freq[pair] * 0.15915494309189535;
      sincosf((float)((turns - floor(turns)) * 6.283185307179586), &sn, &cs);
#endif
      const float a = src[h * hd + 2 * pair], b = src[h * hd + 2 * pair + 1];
      val = (le & 1) ? fmaf(b, cs, a * sn) : fmaf(a, cs, -b * sn);
    }
    if (is_q) qr[e] = from_f32<TA>(val);
    else if (slot >= 0 && kpool != nullptr)
      kpool[(((size_t)page * n_kv_heads + h) * page_size + off) * hd + le] = from_f32<TA>(val);
  }
  if (slot >= 0 && vpool != nullptr) {
    for (int i = threadIdx.x; i < vw; i += blockDim.x) {
      const int h = i / hd_v, le = i - h * hd_v;
      const float x = to_f32(vr[i]) + (v_bias ? to_f32(v_bias[i]) : 0.f);
      vpool[(((size_t)page * n_kv_heads + h) * page_size + off) * hd_v + le] = from_f32<TA>(x);
    }
  }
}

extern "C" int ie_rownorm_rotate_write(void* q, const void* k, const void* v, int q_stride, int k_stride, int v_stride,
                                       const void* q_bias, const void* k_bias, const void* v_bias, const void* q_gain,
                                       const void* k_gain, int w_dtype, float eps, const double* inv_freq, int rot_dims,
                                       const int* positions, const int* slot_mapping, void* kpool, void* vpool,
                                       int n_tokens, int n_heads, int n_kv_heads, int hd, int hd_v, int page_size,
                                       int act_dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (rot_dims < 0 || rot_dims > hd || (rot_dims & 1) || (rot_dims > 0 && inv_freq == nullptr)) return IE_BAD_SIZE;
  const size_t smem = sizeof(float) * (size_t)(n_heads + n_kv_heads) * hd;
  if (smem > 200 * 1024) return IE_BAD_SIZE;
  const int threads = (n_heads * hd) >= 2048 ? 256 : 128;
#define RRW_GO(TA, TW)                                                                                               \
  {                                                                                                                  \
    if (smem > 47 * 1024) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(rownorm_rotate_write_kernel<TA, TW>,                                      \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
      if (e != cudaSuccess) return (int)e;                                                                           \
    }                                                                                                                \
    return launch_k(rownorm_rotate_write_kernel<TA, TW>, n_tokens, threads, smem, stream, (TA*)q, (const TA*)k,      \
                    (const TA*)v, q_stride, k_stride, v_stride, (const TW*)q_bias, (const TW*)k_bias,                \
                    (const TW*)v_bias, (const TW*)q_gain, (const TW*)k_gain, eps, inv_freq, rot_dims, positions,     \
                    slot_mapping, (TA*)kpool, (TA*)vpool, n_heads, n_kv_heads, hd, hd_v, page_size);                 \
  }
  if (act_dtype == IE_F32 && w_dtype == IE_F32) RRW_GO(float, float);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) RRW_GO(float, bf16);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) RRW_GO(bf16, float);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) RRW_GO(bf16, bf16);
#undef RRW_GO
  return IE_BAD_DTYPE;
}

IE_CHECK_API(sequence)
