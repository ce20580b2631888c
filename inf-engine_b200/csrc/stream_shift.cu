// Work on the residual stream and on what a sublayer reads from it.
//
// scale_add_sinusoid: x <- x * scale + s(position), s the sinusoidal position vector of the stream's width:
//     s[2i] = sin(p * base^(-2i / width)),  s[2i + 1] = cos(p * base^(-2i / width))
//   The frequency and its product with the position are formed and brought into one turn in double; sine and cosine
//   are float32.
// add_row: x[n, :] += row, one vector for every token of the step (what a pass of repeated layers adds to the stream).
// token_shift: a sublayer's input h is replaced by h + (h' - h) * mu, coordinate by coordinate, with h' the h of the
//   token before as it was BEFORE this replacement, and zeros before a sequence's first token.  The last h of every
//   request is state (one row a slot): a request's first token of the step reads it, and the thread that read it
//   stores the request's last h of the step in its place, so a cut of the prompt changes nothing.  The difference,
//   the product and the sum are float32.
// gate_mul: x[n, j] *= sigmoid(g[n, j / group]): an output gate per coordinate (group = 1) or per head (group = head
//   size); sigmoid and product in float32.
#include "common.cuh"

// A thread keeps one coordinate and walks SIN_TOKENS tokens: its frequency (a double-precision exponential) is formed once.
#define SIN_TOKENS 16
__global__ void scale_add_sinusoid_kernel(float* __restrict__ x, const int* __restrict__ positions, float scale,
                                          double log_base, int n, int d) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  const double turns_per_position = exp(-log_base * (double)(c & ~1) / (double)d) * 0.15915494309189535;
  const int t_end = min(n, ((int)blockIdx.y + 1) * SIN_TOKENS);
  for (int t = blockIdx.y * SIN_TOKENS; t < t_end; ++t) {
    const double turns = (double)positions[t] * turns_per_position;
    float sn, cs;
    sincosf((float)((turns - floor(turns)) * 6.283185307179586), &sn, &cs);
    float* at = x + (size_t)t * d + c;
    *at = fmaf(*at, scale, (c & 1) ? cs : sn);
  }
}

extern "C" int ie_scale_add_sinusoid(float* x, const int* positions, float scale, double base, int n, int d,
                                     cudaStream_t stream) {
  if (n <= 0 || d <= 0) return IE_OK;
  if (!(base > 0.0)) return IE_BAD_SIZE;
  const int threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
  const dim3 grid((d + threads - 1) / threads, (n + SIN_TOKENS - 1) / SIN_TOKENS);
  if (grid.y > 65535) return IE_BAD_SIZE;
  return launch_k(scale_add_sinusoid_kernel, grid, threads, 0, stream, x, positions, scale, log(base), n, d);
}

template <typename TW>
__global__ void add_row_kernel(float* __restrict__ x, const TW* __restrict__ row, int n, int d) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * d) return;
  x[i] += to_f32(row[i % d]);
}

extern "C" int ie_add_row(float* x, const void* row, int row_dtype, int n, int d, cudaStream_t stream) {
  if (n <= 0 || d <= 0) return IE_OK;
  const unsigned blocks = (unsigned)(((long long)n * d + 255) / 256);
  if (row_dtype == IE_F32) return launch_k(add_row_kernel<float>, blocks, 256, 0, stream, x, (const float*)row, n, d);
  if (row_dtype == IE_BF16) return launch_k(add_row_kernel<bf16>, blocks, 256, 0, stream, x, (const bf16*)row, n, d);
  return IE_BAD_DTYPE;
}

// A block a token (and 1,024 coordinates of it); the token's request is found in q_start by a search.
template <typename TA, typename TW>
__global__ void token_shift_kernel(const TA* __restrict__ h, TA* __restrict__ out, const TW* __restrict__ mu,
                                   TA* __restrict__ state, const int* __restrict__ q_start,
                                   const int* __restrict__ ctx_before, const int* __restrict__ slots, int n_requests,
                                   int d, int write_state) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int lo = 0, hi = n_requests;                     // the request r with q_start[r] <= t < q_start[r + 1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (q_start[mid] <= t) lo = mid; else hi = mid;
  }
  const int t0 = q_start[lo], t1 = q_start[lo + 1];
  const bool first = t == t0;
  const int slot = IE_SLOT(slots[lo]);
  TA* srow = slot >= 0 ? state + (size_t)slot * d : nullptr;
  const bool from_state = first && ctx_before[lo] > 0 && srow != nullptr;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < d; c += gridDim.y * blockDim.x) {
    const float cur = to_f32(h[(size_t)t * d + c]);
    float prev = 0.f;
    if (!first) prev = to_f32(h[(size_t)(t - 1) * d + c]);
    else if (from_state) prev = to_f32(srow[c]);
    if (first && write_state && srow != nullptr) srow[c] = h[(size_t)(t1 - 1) * d + c];
    out[(size_t)t * d + c] = from_f32<TA>(fmaf(prev - cur, to_f32(mu[c]), cur));
  }
}

// bfloat16 rows whose width is a multiple of 8: a thread takes 16 bytes of a row; the token's request is found by one
// load a lane and a vote (requests beyond 32: a loop of such votes), not by a chain of dependent loads
__device__ __forceinline__ int request_of_token(const int* __restrict__ q_start, int n_requests, int t) {
  const int lane = threadIdx.x & 31;
  int count = 0;
  for (int r0 = 0; r0 < n_requests; r0 += 32) {
    const int r = r0 + lane;
    count += __popc(__ballot_sync(0xffffffffu, r < n_requests && q_start[r] <= t));
  }
  return count - 1;
}

template <typename TW>
__global__ void token_shift_vec_kernel(const bf16* __restrict__ h, bf16* __restrict__ out, const TW* __restrict__ mu,
                                       bf16* __restrict__ state, const int* __restrict__ q_start,
                                       const int* __restrict__ ctx_before, const int* __restrict__ slots, int n_requests,
                                       int d, int write_state) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int lo = request_of_token(q_start, n_requests, t);
  const int t0 = q_start[lo], t1 = q_start[lo + 1];
  const bool first = t == t0;
  const int slot = IE_SLOT(slots[lo]);
  bf16* srow = slot >= 0 ? state + (size_t)slot * d : nullptr;
  const bool from_state = first && ctx_before[lo] > 0 && srow != nullptr;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < d; c += gridDim.y * blockDim.x * 8) {
    const uint4 cur = *reinterpret_cast<const uint4*>(h + (size_t)t * d + c);
    uint4 prev = make_uint4(0u, 0u, 0u, 0u);
    if (!first) prev = *reinterpret_cast<const uint4*>(h + (size_t)(t - 1) * d + c);
    else if (from_state) prev = *reinterpret_cast<const uint4*>(srow + c);
    if (first && write_state && srow != nullptr)
      *reinterpret_cast<uint4*>(srow + c) = *reinterpret_cast<const uint4*>(h + (size_t)(t1 - 1) * d + c);
    const __nv_bfloat162* cp = reinterpret_cast<const __nv_bfloat162*>(&cur);
    const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&prev);
    uint4 res;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 cf = __bfloat1622float2(cp[j]), pf = __bfloat1622float2(pp[j]);
      rp[j] = __floats2bfloat162_rn(fmaf(pf.x - cf.x, to_f32(mu[c + 2 * j]), cf.x),
                                    fmaf(pf.y - cf.y, to_f32(mu[c + 2 * j + 1]), cf.y));
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * d + c) = res;
  }
}

extern "C" int ie_token_shift(const void* h, void* out, int act_dtype, const void* mu, int mu_dtype, void* state,
                              const int* q_start, const int* ctx_before, const int* slots, int n_requests, int n, int d,
                              int write_state, cudaStream_t stream) {
  if (n <= 0 || d <= 0 || n_requests <= 0) return IE_OK;
  if (h == out) return IE_BAD_SIZE;                // a token reads the row before it as it was
  if (act_dtype == IE_BF16 && (d & 7) == 0 && ((((uintptr_t)h) | ((uintptr_t)out) | ((uintptr_t)state)) & 15) == 0) {
    const int threads = d / 8 >= 256 ? 256 : ((d / 8 + 31) / 32) * 32;
    dim3 vgrid(n, (d / 8 + threads - 1) / threads);
    if (mu_dtype == IE_F32)
      return launch_k(token_shift_vec_kernel<float>, vgrid, threads, 0, stream, (const bf16*)h, (bf16*)out, (const float*)mu,
                      (bf16*)state, q_start, ctx_before, slots, n_requests, d, write_state);
    if (mu_dtype == IE_BF16)
      return launch_k(token_shift_vec_kernel<bf16>, vgrid, threads, 0, stream, (const bf16*)h, (bf16*)out, (const bf16*)mu,
                      (bf16*)state, q_start, ctx_before, slots, n_requests, d, write_state);
  }
  dim3 grid(n, (d + 1023) / 1024);
#define TS_GO(TA, TW)                                                                                              \
  return launch_k(token_shift_kernel<TA, TW>, grid, 256, 0, stream, (const TA*)h, (TA*)out, (const TW*)mu, (TA*)state, \
                  q_start, ctx_before, slots, n_requests, d, write_state)
  if (act_dtype == IE_F32 && mu_dtype == IE_F32) TS_GO(float, float);
  if (act_dtype == IE_F32 && mu_dtype == IE_BF16) TS_GO(float, bf16);
  if (act_dtype == IE_BF16 && mu_dtype == IE_F32) TS_GO(bf16, float);
  if (act_dtype == IE_BF16 && mu_dtype == IE_BF16) TS_GO(bf16, bf16);
#undef TS_GO
  return IE_BAD_DTYPE;
}

template <typename TA>
__global__ void gate_mul_kernel(TA* __restrict__ x, int x_stride, const TA* __restrict__ g, int g_stride, int n, int d,
                                int group) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * d) return;
  const int t = (int)(i / d), c = (int)(i - (long long)t * d);
  const float z = to_f32(g[(size_t)t * g_stride + c / group]);
  TA* at = x + (size_t)t * x_stride + c;
  *at = from_f32<TA>(to_f32(*at) / (1.f + expf(-z)));
}

// bfloat16 rows in 16-byte pieces: a gate per coordinate (eight of them loaded together) or one gate for the eight
__global__ void gate_mul_vec_kernel(bf16* __restrict__ x, int x_stride, const bf16* __restrict__ g, int g_stride, int n,
                                    int d, int group) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = d >> 3;
  if (i >= (long long)n * per_row) return;
  const int t = (int)(i / per_row), c = (int)(i - (long long)t * per_row) << 3;
  bf16* at = x + (size_t)t * x_stride + c;
  const uint4 raw = *reinterpret_cast<const uint4*>(at);
  const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float z[8];
  if (group == 1) {
    const uint4 gr = *reinterpret_cast<const uint4*>(g + (size_t)t * g_stride + c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gr);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(gp[j]);
      z[2 * j] = f.x;
      z[2 * j + 1] = f.y;
    }
  } else {
    const float one = to_f32(g[(size_t)t * g_stride + c / group]);
#pragma unroll
    for (int j = 0; j < 8; ++j) z[j] = one;
  }
  uint4 res;
  __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(xp[j]);
    rp[j] = __floats2bfloat162_rn(f.x / (1.f + expf(-z[2 * j])), f.y / (1.f + expf(-z[2 * j + 1])));
  }
  *reinterpret_cast<uint4*>(at) = res;
}

extern "C" int ie_gate_mul(void* x, int x_stride, const void* g, int g_stride, int n, int d, int group, int act_dtype,
                           cudaStream_t stream) {
  if (n <= 0 || d <= 0) return IE_OK;
  if (group <= 0 || d % group) return IE_BAD_SIZE;
  if (act_dtype == IE_BF16 && (d & 7) == 0 && (x_stride & 7) == 0 && (((uintptr_t)x) & 15) == 0 &&
      (group == 1 ? ((g_stride & 7) == 0 && (((uintptr_t)g) & 15) == 0) : (group & 7) == 0))
    return launch_k(gate_mul_vec_kernel, (unsigned)(((long long)n * (d >> 3) + 255) / 256), 256, 0, stream, (bf16*)x, x_stride,
                    (const bf16*)g, g_stride, n, d, group);
  const unsigned blocks = (unsigned)(((long long)n * d + 255) / 256);
  if (act_dtype == IE_F32)
    return launch_k(gate_mul_kernel<float>, blocks, 256, 0, stream, (float*)x, x_stride, (const float*)g, g_stride, n, d, group);
  if (act_dtype == IE_BF16)
    return launch_k(gate_mul_kernel<bf16>, blocks, 256, 0, stream, (bf16*)x, x_stride, (const bf16*)g, g_stride, n, d, group);
  return IE_BAD_DTYPE;
}

IE_CHECK_API(stream_shift)
