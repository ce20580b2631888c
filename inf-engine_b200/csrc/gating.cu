// Gates: element-by-element kernels of layers that gate what they add, and a gated recurrence without a hidden-state
// input to its gates.  All arithmetic is float32 whatever the storage type.
//
// gated_residual_add:  residual += sigmoid(gate_pre + bias) * y          (residual float32; a gate per coordinate)
// scale_rows:          x *= scale, and a copy of the result where asked   (a scaled embedding that is used again later)
// glu_act:             out = act(g) * (u + up_offset) over rows that hold gate and up side by side or alternating:
//                      kind 0: g * sigmoid(g);  kind 1: g' * sigmoid(alpha g') with g' = min(g, limit) and u clamped to
//                      [-limit, limit]
// mingru_scan:         z = sigmoid(z_pre + z_bias), u = u_pre + u_bias, candidate = u + 1/2 (u >= 0) | sigmoid(u) (u < 0)
//                      S <- S + z (candidate - S)   [= (1 - z) S + z candidate],  out = S * silu(g_pre)
//                      per channel, over each request's tokens of the step in order, from the float32 state of the
//                      request's slot (negative slot: a padding row, skipped)
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

template <typename T, typename TB>
__global__ void gated_residual_add_kernel(float* __restrict__ residual, const T* __restrict__ y, int y_stride,
                                          const T* __restrict__ gate, int gate_stride, const TB* __restrict__ bias,
                                          int n_rows, int d) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_rows * d) return;
  const int r = (int)(i / d), c = (int)(i - (size_t)r * d);
  const float g = to_f32(gate[(size_t)r * gate_stride + c]) + (bias != nullptr ? to_f32(bias[c]) : 0.f);
  residual[i] = fmaf(sigmoid_f(g), to_f32(y[(size_t)r * y_stride + c]), residual[i]);
}

// bfloat16 rows whose width and strides are multiples of 8: eight coordinates a thread, 16-byte loads and stores
template <typename TB>
__global__ void gated_residual_add_bf16_vec_kernel(float* __restrict__ residual, const bf16* __restrict__ y, int y_stride,
                                                   const bf16* __restrict__ gate, int gate_stride,
                                                   const TB* __restrict__ bias, size_t n_vec, int d8) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const size_t r = i / d8;
  const int c = (int)(i - r * d8) * 8;
  const uint4 yv = *reinterpret_cast<const uint4*>(y + r * y_stride + c);
  const uint4 gv = *reinterpret_cast<const uint4*>(gate + r * gate_stride + c);
  const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&yv);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
  float4* res = reinterpret_cast<float4*>(residual + r * (size_t)d8 * 8 + c);
  float4 a = res[0], b = res[1];
  float* out[2] = {&a.x, &b.x};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 yf = __bfloat1622float2(y2[k]), gf = __bfloat1622float2(g2[k]);
    const float b0 = bias != nullptr ? to_f32(bias[c + 2 * k]) : 0.f, b1 = bias != nullptr ? to_f32(bias[c + 2 * k + 1]) : 0.f;
    float* o = out[k >> 1] + 2 * (k & 1);
    o[0] = fmaf(sigmoid_f(gf.x + b0), yf.x, o[0]);
    o[1] = fmaf(sigmoid_f(gf.y + b1), yf.y, o[1]);
  }
  res[0] = a;
  res[1] = b;
}

extern "C" int ie_gated_residual_add(float* residual, const void* y, int y_stride, const void* gate, int gate_stride,
                                     const void* bias, int bias_dtype, int n_rows, int d, int act_dtype,
                                     cudaStream_t stream) {
  const size_t n = (size_t)n_rows * d;
  if (n == 0) return IE_OK;
  if (act_dtype == IE_BF16 && d % 8 == 0 && y_stride % 8 == 0 && gate_stride % 8 == 0 &&
      (((uintptr_t)residual | (uintptr_t)y | (uintptr_t)gate) & 15) == 0) {
    const size_t n_vec = n / 8;
    const unsigned vblocks = (unsigned)((n_vec + 255) / 256);
    if (bias_dtype == IE_F32)
      return launch_k(gated_residual_add_bf16_vec_kernel<float>, vblocks, 256, 0, stream, residual, (const bf16*)y, y_stride,
                      (const bf16*)gate, gate_stride, (const float*)bias, n_vec, d / 8);
    if (bias_dtype == IE_BF16)
      return launch_k(gated_residual_add_bf16_vec_kernel<bf16>, vblocks, 256, 0, stream, residual, (const bf16*)y, y_stride,
                      (const bf16*)gate, gate_stride, (const bf16*)bias, n_vec, d / 8);
    return IE_BAD_DTYPE;
  }
  const unsigned blocks = (unsigned)((n + 255) / 256);
#define GR_GO(T, TB)                                                                                             \
  return launch_k(gated_residual_add_kernel<T, TB>, blocks, 256, 0, stream, residual, (const T*)y, y_stride,     \
                  (const T*)gate, gate_stride, (const TB*)bias, n_rows, d)
  if (act_dtype == IE_F32 && bias_dtype == IE_F32) GR_GO(float, float);
  if (act_dtype == IE_F32 && bias_dtype == IE_BF16) GR_GO(float, bf16);
  if (act_dtype == IE_BF16 && bias_dtype == IE_F32) GR_GO(bf16, float);
  if (act_dtype == IE_BF16 && bias_dtype == IE_BF16) GR_GO(bf16, bf16);
#undef GR_GO
  return IE_BAD_DTYPE;
}

__global__ void scale_rows_kernel(float* __restrict__ x, float* __restrict__ keep, float scale, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = x[i] * scale;
  x[i] = v;
  if (keep != nullptr) keep[i] = v;
}

extern "C" int ie_scale_rows(float* x, float* keep, float scale, int n_rows, int d, cudaStream_t stream) {
  const size_t n = (size_t)n_rows * d;
  if (n == 0) return IE_OK;
  return launch_k(scale_rows_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, keep, scale, n);
}

template <typename T>
__global__ void glu_act_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, int in_stride, size_t total,
                               int interleaved, int kind, float alpha, float limit, float up_offset) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int r = (int)(i / inter), j = (int)(i - (size_t)r * inter);
  const T* row = in + (size_t)r * in_stride;
  float g = to_f32(interleaved ? row[2 * j] : row[j]);
  float u = to_f32(interleaved ? row[2 * j + 1] : row[inter + j]);
  float a;
  if (kind == 1) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    a = g * sigmoid_f(alpha * g);
  } else {
    a = g * sigmoid_f(g);
  }
  out[i] = from_f32<T>(a * (u + up_offset));
}

// bfloat16, eight outputs a thread (inter and the row stride multiples of 8, rows that start on 16 bytes)
__global__ void glu_act_bf16_vec_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int inter, int in_stride,
                                        size_t total8, int interleaved, int kind, float alpha, float limit, float up_offset) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int per_row = inter >> 3;
  const size_t n = idx / per_row;
  const int j = (int)(idx - n * per_row) * 8;
  const bf16* row = in + n * in_stride;
  float g[8], u[8];
  const uint4 a = *reinterpret_cast<const uint4*>(interleaved ? row + 2 * j : row + j);
  const uint4 b = *reinterpret_cast<const uint4*>(interleaved ? row + 2 * j + 8 : row + inter + j);
  const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 x = __bfloat1622float2(ap[t]), y = __bfloat1622float2(bp[t]);
    if (interleaved) {
      g[t] = x.x; u[t] = x.y; g[4 + t] = y.x; u[4 + t] = y.y;
    } else {
      g[2 * t] = x.x; g[2 * t + 1] = x.y; u[2 * t] = y.x; u[2 * t + 1] = y.y;
    }
  }
  float r[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    float gg = g[t], uu = u[t], act;
    if (kind == 1) {
      gg = fminf(gg, limit);
      uu = fminf(fmaxf(uu, -limit), limit);
      act = gg * sigmoid_f(alpha * gg);
    } else {
      act = gg * sigmoid_f(gg);
    }
    r[t] = act * (uu + up_offset);
  }
  uint4 o;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int t = 0; t < 4; ++t) op[t] = __floats2bfloat162_rn(r[2 * t], r[2 * t + 1]);
  *reinterpret_cast<uint4*>(out + n * inter + j) = o;
}

extern "C" int ie_glu_act(const void* in, void* out, int n_rows, int inter, int in_stride, int interleaved, int kind,
                          float alpha, float limit, float up_offset, int act_dtype, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * inter;
  if (total == 0) return IE_OK;
  if (kind < 0 || kind > 1) return IE_BAD_SIZE;
  if (act_dtype == IE_BF16 && inter % 8 == 0 && in_stride % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
    const size_t total8 = total / 8;
    return launch_k(glu_act_bf16_vec_kernel, (unsigned)((total8 + 255) / 256), 256, 0, stream, (const bf16*)in, (bf16*)out,
                    inter, in_stride, total8, interleaved, kind, alpha, limit, up_offset);
  }
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (act_dtype == IE_F32)
    return launch_k(glu_act_kernel<float>, blocks, 256, 0, stream, (const float*)in, (float*)out, inter, in_stride, total,
                    interleaved, kind, alpha, limit, up_offset);
  if (act_dtype == IE_BF16)
    return launch_k(glu_act_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)in, (bf16*)out, inter, in_stride, total,
                    interleaved, kind, alpha, limit, up_offset);
  return IE_BAD_DTYPE;
}

#define MG_UNROLL 4

template <typename T, typename TB>
__global__ void mingru_scan_kernel(const T* __restrict__ z_pre, const T* __restrict__ u_pre, int zu_stride,
                                   const T* __restrict__ g_pre, int g_stride, const TB* __restrict__ z_bias,
                                   const TB* __restrict__ u_bias, float* __restrict__ state, T* __restrict__ out,
                                   int out_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
                                   int width, int write_state) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int slot = IE_SLOT(slots[r]);
  if (slot < 0) return;
  const int t0 = q_start[r], t1 = q_start[r + 1];
  const float bz = z_bias != nullptr ? to_f32(z_bias[c]) : 0.f, bu = u_bias != nullptr ? to_f32(u_bias[c]) : 0.f;
  float S = state[(size_t)slot * width + c];
  for (int t = t0; t < t1; t += MG_UNROLL) {
    float zp[MG_UNROLL], up[MG_UNROLL], gp[MG_UNROLL];
#pragma unroll
    for (int i = 0; i < MG_UNROLL; ++i) {        // the loads of a few tokens on their way together: none depends on S
      const bool live = t + i < t1;
      const size_t row = (size_t)(live ? t + i : t);
      zp[i] = to_f32(z_pre[row * zu_stride + c]);
      up[i] = to_f32(u_pre[row * zu_stride + c]);
      gp[i] = to_f32(g_pre[row * g_stride + c]);
    }
#pragma unroll
    for (int i = 0; i < MG_UNROLL; ++i) {
      if (t + i < t1) {
        const float z = sigmoid_f(zp[i] + bz);
        const float u = up[i] + bu;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        S = fmaf(z, cand - S, S);
        out[(size_t)(t + i) * out_stride + c] = from_f32<T>(S * (gp[i] * sigmoid_f(gp[i])));
      }
    }
  }
  if (write_state) state[(size_t)slot * width + c] = S;
}

// The same recurrence for requests that bring many tokens (prompt portions).  The recurrence is linear in the state,
// S_t = (1 - z_t) S_(t-1) + z_t c_t, so a run of tokens maps the state it starts from to A S + B with A = prod (1 - z_t)
// and B the run's result from a zero state.  A block takes MGS_CH channels of one request and cuts its tokens into
// MGS_SEG runs, a thread a (channel, run): pass one forms every run's (A, B), the first run's threads then carry the
// state through the MGS_SEG pairs, pass two repeats every run from its true starting state and writes the outputs.
// Twice the arithmetic and reads (the second time from cache) for a dependent chain of T / MGS_SEG + MGS_SEG steps.
#define MGS_CH 32
#define MGS_SEG 32

template <typename T, typename TB>
__global__ void __launch_bounds__(MGS_CH * MGS_SEG) mingru_scan_segments_kernel(
    const T* __restrict__ z_pre, const T* __restrict__ u_pre, int zu_stride, const T* __restrict__ g_pre, int g_stride,
    const TB* __restrict__ z_bias, const TB* __restrict__ u_bias, float* __restrict__ state, T* __restrict__ out,
    int out_stride, const int* __restrict__ q_start, const int* __restrict__ slots, int width, int write_state) {
  __shared__ float sA[MGS_SEG][MGS_CH], sB[MGS_SEG][MGS_CH];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int slot = IE_SLOT(slots[r]);
  if (slot < 0) return;                              // (the whole block)
  const int cx = threadIdx.x, sg = threadIdx.y;
  const int c = blockIdx.x * MGS_CH + cx;
  const bool live = c < width;
  const int cc = live ? c : width - 1;
  const int t0 = q_start[r], t1 = q_start[r + 1];
  const int seg_len = (t1 - t0 + MGS_SEG - 1) / MGS_SEG;
  const int a = min(t1, t0 + sg * seg_len), b = min(t1, a + seg_len);
  const float bz = z_bias != nullptr ? to_f32(z_bias[cc]) : 0.f, bu = u_bias != nullptr ? to_f32(u_bias[cc]) : 0.f;
  float A = 1.f, B = 0.f;
  for (int t = a; t < b; t += MG_UNROLL) {
    float zp[MG_UNROLL], up[MG_UNROLL];
#pragma unroll
    for (int i = 0; i < MG_UNROLL; ++i) {
      const size_t row = (size_t)(t + i < b ? t + i : t);
      zp[i] = to_f32(z_pre[row * zu_stride + cc]);
      up[i] = to_f32(u_pre[row * zu_stride + cc]);
    }
#pragma unroll
    for (int i = 0; i < MG_UNROLL; ++i) {
      if (t + i < b) {
        const float z = sigmoid_f(zp[i] + bz);
        const float u = up[i] + bu;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        A *= 1.f - z;
        B = fmaf(z, cand - B, B);
      }
    }
  }
  sA[sg][cx] = A;
  sB[sg][cx] = B;
  __syncthreads();
  if (sg == 0) {
    float S = state[(size_t)slot * width + cc];
    for (int k = 0; k < MGS_SEG; ++k) {
      const float a_k = sA[k][cx], b_k = sB[k][cx];
      sA[k][cx] = S;                                 // the state that run k starts from
      S = fmaf(a_k, S, b_k);
    }
    if (write_state && live) state[(size_t)slot * width + c] = S;
  }
  __syncthreads();
  float S = sA[sg][cx];
  for (int t = a; t < b; t += MG_UNROLL) {
    float zp[MG_UNROLL], up[MG_UNROLL], gp[MG_UNROLL];
#pragma unroll
    for (int i = 0; i < MG_UNROLL; ++i) {
      const size_t row = (size_t)(t + i < b ? t + i : t);
      zp[i] = to_f32(z_pre[row * zu_stride + cc]);
      up[i] = to_f32(u_pre[row * zu_stride + cc]);
      gp[i] = to_f32(g_pre[row * g_stride + cc]);
    }
#pragma unroll
    for (int i = 0; i < MG_UNROLL; ++i) {
      if (t + i < b) {
        const float z = sigmoid_f(zp[i] + bz);
        const float u = up[i] + bu;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        S = fmaf(z, cand - S, S);
        if (live) out[(size_t)(t + i) * out_stride + c] = from_f32<T>(S * (gp[i] * sigmoid_f(gp[i])));
      }
    }
  }
}

// max_q_len: the most tokens a request of the step brings, if the host knows (0: it does not); from MGS_MIN_TOKENS on the
// kernel that cuts each request's tokens into runs is launched
#define MGS_MIN_TOKENS 64

extern "C" int ie_mingru_scan_hint(const void* z_pre, const void* u_pre, int zu_stride, const void* g_pre, int g_stride,
                                   const void* z_bias, const void* u_bias, int bias_dtype, float* state, void* out,
                                   int out_stride, const int* q_start, const int* slots, int n_requests, int width,
                                   int write_state, int act_dtype, int max_q_len, cudaStream_t stream);

extern "C" int ie_mingru_scan(const void* z_pre, const void* u_pre, int zu_stride, const void* g_pre, int g_stride,
                              const void* z_bias, const void* u_bias, int bias_dtype, float* state, void* out,
                              int out_stride, const int* q_start, const int* slots, int n_requests, int width,
                              int write_state, int act_dtype, cudaStream_t stream) {
  return ie_mingru_scan_hint(z_pre, u_pre, zu_stride, g_pre, g_stride, z_bias, u_bias, bias_dtype, state, out, out_stride,
                             q_start, slots, n_requests, width, write_state, act_dtype, 0, stream);
}

extern "C" int ie_mingru_scan_hint(const void* z_pre, const void* u_pre, int zu_stride, const void* g_pre, int g_stride,
                              const void* z_bias, const void* u_bias, int bias_dtype, float* state, void* out,
                                   int out_stride, const int* q_start, const int* slots, int n_requests, int width,
                                   int write_state, int act_dtype, int max_q_len, cudaStream_t stream) {
  if (n_requests <= 0 || width <= 0) return IE_OK;
  if (n_requests > 65535) return IE_BAD_SIZE;
  if (max_q_len >= MGS_MIN_TOKENS) {
    const dim3 sgrid((width + MGS_CH - 1) / MGS_CH, n_requests), sblock(MGS_CH, MGS_SEG);
#define MGS_GO(T, TB)                                                                                                    \
  return launch_k(mingru_scan_segments_kernel<T, TB>, sgrid, sblock, 0, stream, (const T*)z_pre, (const T*)u_pre, zu_stride, \
                  (const T*)g_pre, g_stride, (const TB*)z_bias, (const TB*)u_bias, state, (T*)out, out_stride, q_start,     \
                  slots, width, write_state)
    if (act_dtype == IE_F32 && bias_dtype == IE_F32) MGS_GO(float, float);
    if (act_dtype == IE_F32 && bias_dtype == IE_BF16) MGS_GO(float, bf16);
    if (act_dtype == IE_BF16 && bias_dtype == IE_F32) MGS_GO(bf16, float);
    if (act_dtype == IE_BF16 && bias_dtype == IE_BF16) MGS_GO(bf16, bf16);
#undef MGS_GO
    return IE_BAD_DTYPE;
  }
  const int threads = 64;
  dim3 grid((width + threads - 1) / threads, n_requests);
#define MG_GO(T, TB)                                                                                              \
  return launch_k(mingru_scan_kernel<T, TB>, grid, threads, 0, stream, (const T*)z_pre, (const T*)u_pre, zu_stride, \
                  (const T*)g_pre, g_stride, (const TB*)z_bias, (const TB*)u_bias, state, (T*)out, out_stride,     \
                  q_start, slots, width, write_state)
  if (act_dtype == IE_F32 && bias_dtype == IE_F32) MG_GO(float, float);
  if (act_dtype == IE_F32 && bias_dtype == IE_BF16) MG_GO(float, bf16);
  if (act_dtype == IE_BF16 && bias_dtype == IE_F32) MG_GO(bf16, float);
  if (act_dtype == IE_BF16 && bias_dtype == IE_BF16) MG_GO(bf16, bf16);
#undef MG_GO
  return IE_BAD_DTYPE;
}

IE_CHECK_API(gating)
