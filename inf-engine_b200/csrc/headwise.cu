// Work on the heads of a token's projections, before and after attention.
//
// head_prepare: for every token, on the query side and on the key side, each with its own head count and head size:
//   * an optional RMS norm over the FIRST `norm_dims` dimensions of every head (x / sqrt(mean(x^2) + eps) * gain, gain of
//     that size, shared by the heads; the other dimensions pass unchanged): a norm of whole heads when norm_dims is the
//     head size, a norm of the compressed part of a key row that also carries a rotated part when it is less;
//   * a rotation by position of `rot_dims` dimensions that start at dimension `rot_off` of every head, either in halves
//     (dimension i with i + rot_dims / 2) or in neighbouring pairs (2i with 2i + 1):
//         (u, v) -> (u cos a - v sin a, v cos a + u sin a) * mult,  a = position * inv_freq[i]
//     inv_freq is float64 (blended frequencies of a scaled rotation are worked out on the host), the product with the
//     position is formed and brought into one turn in double, sine and cosine are float32;
//   * queries are written back in place, keys go to their page slot in a pool [page, key heads, page_size, head size]
//     and values (optional, copied as they are) to [page, value heads, page_size, value size].
// A token whose slot is negative (padding) writes nothing to the pools.
//
// heads_gemm: a product per head, out[m, h, j] = sum_k x[m, h, k] * w[h, k, j], float32 products summed in ascending k
// (the same for a row whatever else is in the batch), any of float32 and bfloat16 for x, w and out.
//
// diff_combine: two attention maps of a head that share their values become one output:
//   o = a1 - lambda * a2;  o <- o / sqrt(mean(o^2) + eps) * out_mult * sigmoid(gate)      (gate optional)
#include "common.cuh"

struct HeadSide {
  void* x;            // [n, heads * hd] rows, row stride `stride`
  int stride, heads, hd, norm_dims, rot_off;
  const void* gain;   // [norm_dims] or null
};

template <typename TA, typename TW>
__global__ void head_prepare_kernel(HeadSide qs_, HeadSide ks_, const TA* __restrict__ v, int v_stride, float eps,
                                    const double* __restrict__ inv_freq, int rot_dims, int neighbours, float mult,
                                    const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                    TA* __restrict__ kpool, TA* __restrict__ vpool, int n_v_heads, int hd_v,
                                    int page_size) {
  extern __shared__ float rows[];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int qw = qs_.heads * qs_.hd, kw = ks_.heads * ks_.hd;
  float* sq = rows;
  float* sk = rows + qw;
  TA* qr = (TA*)qs_.x + (size_t)n * qs_.stride;
  TA* kr = (TA*)ks_.x + (size_t)n * ks_.stride;
  for (int i = threadIdx.x; i < qw; i += blockDim.x) sq[i] = to_f32(qr[i]);
  for (int i = threadIdx.x; i < kw; i += blockDim.x) sk[i] = to_f32(kr[i]);
  __syncthreads();
  // norms: a warp a head
  for (int side = 0; side < 2; ++side) {
    const HeadSide& s = side ? ks_ : qs_;
    if (s.gain == nullptr || s.norm_dims <= 0) continue;
    float* base = side ? sk : sq;
    const TW* gain = (const TW*)s.gain;
    for (int h = warp; h < s.heads; h += n_warps) {
      float* hx = base + h * s.hd;
      float ss = 0.f;
      for (int d = lane; d < s.norm_dims; d += 32) ss = fmaf(hx[d], hx[d], ss);
      ss = warp_sum(ss);
      const float r = sqrtf(ss / (float)s.norm_dims + eps);
      for (int d = lane; d < s.norm_dims; d += 32) hx[d] = hx[d] / r * to_f32(gain[d]);
    }
  }
  __syncthreads();
  const double pos = (double)positions[n];
  const int slot = slot_mapping ? IE_SLOT(slot_mapping[n]) : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const int half = rot_dims >> 1;
  for (int i = threadIdx.x; i < qw + kw; i += blockDim.x) {
    const bool is_q = i < qw;
    const HeadSide& s = is_q ? qs_ : ks_;
    const int e = is_q ? i : i - qw;
    const float* src = is_q ? sq : sk;
    const int h = e / s.hd, le = e - h * s.hd;
    float val = src[e];
    const int rd = le - s.rot_off;
    if (inv_freq != nullptr && rd >= 0 && rd < rot_dims) {
      int pair, first;          // which frequency, and whether this is the pair's first member
      int ia, ib;
      if (neighbours) {
        pair = rd >> 1; first = !(rd & 1);
        ia = 2 * pair; ib = ia + 1;
      } else {
        pair = rd < half ? rd : rd - half; first = rd < half;
        ia = pair; ib = pair + half;
      }
      const double turns = pos * inv_freq[pair] * 0.15915494309189535;
      float sn, cs;
      sincosf((float)((turns - floor(turns)) * 6.283185307179586), &sn, &cs);
      const float a = src[h * s.hd + s.rot_off + ia], b = src[h * s.hd + s.rot_off + ib];
      val = (first ? fmaf(a, cs, -b * sn) : fmaf(b, cs, a * sn)) * mult;
    }
    if (is_q) {
      qr[e] = from_f32<TA>(val);
    } else if (slot >= 0 && kpool != nullptr) {
      kpool[(((size_t)page * s.heads + h) * page_size + off) * s.hd + le] = from_f32<TA>(val);
    }
  }
  if (slot >= 0 && vpool != nullptr && v != nullptr) {
    const TA* vr = v + (size_t)n * v_stride;
    const int vw = n_v_heads * hd_v;
    for (int i = threadIdx.x; i < vw; i += blockDim.x) {
      const int h = i / hd_v, le = i - h * hd_v;
      vpool[(((size_t)page * n_v_heads + h) * page_size + off) * hd_v + le] = vr[i];
    }
  }
}

extern "C" int ie_head_prepare(void* q, int q_stride, int q_heads, int q_hd, int q_norm_dims, int q_rot_off,
                               const void* q_gain, void* k, int k_stride, int k_heads, int k_hd, int k_norm_dims,
                               int k_rot_off, const void* k_gain, int w_dtype, const void* v, int v_stride,
                               int n_v_heads, int hd_v, float eps, const double* inv_freq, int rot_dims, int neighbours,
                               float mult, const int* positions, const int* slot_mapping, void* kpool, void* vpool,
                               int n_tokens, int page_size, int act_dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (q_heads < 0 || k_heads < 0 || q_hd <= 0 || k_hd <= 0 || page_size <= 0) return IE_BAD_SIZE;
  if (rot_dims < 0 || (rot_dims & 1)) return IE_BAD_SIZE;
  if (inv_freq != nullptr && (q_rot_off < 0 || k_rot_off < 0 || q_rot_off + rot_dims > q_hd || k_rot_off + rot_dims > k_hd))
    return IE_BAD_SIZE;
  if (q_norm_dims > q_hd || k_norm_dims > k_hd) return IE_BAD_SIZE;
  HeadSide qs{q, q_stride, q_heads, q_hd, q_norm_dims, q_rot_off, q_gain};
  HeadSide ks{k, k_stride, k_heads, k_hd, k_norm_dims, k_rot_off, k_gain};
  const size_t smem = sizeof(float) * ((size_t)q_heads * q_hd + (size_t)k_heads * k_hd);
  if (smem > 200 * 1024) return IE_BAD_SIZE;
  const int threads = 256;
#define HP_GO(TA, TW)                                                                                              \
  {                                                                                                                \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(head_prepare_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                            \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    return launch_k(head_prepare_kernel<TA, TW>, n_tokens, threads, smem, stream, qs, ks, (const TA*)v, v_stride,  \
                    eps, inv_freq, rot_dims, neighbours, mult, positions, slot_mapping, (TA*)kpool, (TA*)vpool,    \
                    n_v_heads, hd_v, page_size);                                                                   \
  }
  if (act_dtype == IE_F32 && w_dtype == IE_F32) HP_GO(float, float);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) HP_GO(float, bf16);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) HP_GO(bf16, float);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) HP_GO(bf16, bf16);
#undef HP_GO
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ a product per head
#define HG_ROWS 8
#define HG_THREADS 128

// A block takes `groups` x HG_ROWS rows of one head: its threads are `groups` row groups of blockDim.x / groups columns,
// so that a narrow output (fewer columns than threads) still keeps every thread busy.  Block z takes the columns
// z * z_cols .. (z + 1) * z_cols - 1: a few rows (decode tokens) are spread over many small blocks, a column each thread.
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(HG_THREADS) heads_gemm_kernel(const TX* __restrict__ x, int x_stride, int x_head,
                                                                const TW* __restrict__ w, TO* __restrict__ out,
                                                                int o_stride, int o_head, int M, int K, int N, int groups,
                                                                int z_cols) {
  extern __shared__ float xs[];          // [groups * HG_ROWS][K]
  pdl_trigger();
  pdl_wait();
  const int threads = blockDim.x;
  const int block_rows = groups * HG_ROWS, cols = threads / groups;
  const int m0 = blockIdx.x * block_rows, h = blockIdx.y;
  const int rows = min(block_rows, M - m0);
  for (int i = threadIdx.x; i < block_rows * K; i += threads) {
    const int r = i / K, k = i - r * K;
    xs[i] = r < rows ? to_f32(x[(size_t)(m0 + r) * x_stride + h * x_head + k]) : 0.f;
  }
  __syncthreads();
  const TW* wh = w + (size_t)h * K * N;
  const int rg = threadIdx.x / cols, r0 = rg * HG_ROWS;
  const float* xg = xs + (size_t)r0 * K;
  const int j_end = min(N, ((int)blockIdx.z + 1) * z_cols);
  for (int j = (int)blockIdx.z * z_cols + threadIdx.x - rg * cols; j < j_end; j += cols) {
    float acc[HG_ROWS];
#pragma unroll
    for (int r = 0; r < HG_ROWS; ++r) acc[r] = 0.f;
#pragma unroll 8
    for (int k = 0; k < K; ++k) {
      const float wv = to_f32(wh[(size_t)k * N + j]);
#pragma unroll
      for (int r = 0; r < HG_ROWS; ++r) acc[r] = fmaf(xg[r * K + k], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < HG_ROWS; ++r)
      if (r0 + r < rows) out[(size_t)(m0 + r0 + r) * o_stride + h * o_head + j] = from_f32<TO>(acc[r]);
  }
}

extern "C" int ie_heads_gemm(const void* x, int x_dtype, int x_stride, int x_head, const void* w, int w_dtype, void* out,
                             int o_dtype, int o_stride, int o_head, int M, int H, int K, int N, cudaStream_t stream) {
  if (M <= 0 || H <= 0 || N <= 0) return IE_OK;
  if (K <= 0 || H > 65535) return IE_BAD_SIZE;
  // narrow outputs and enough rows: two or four row groups a block (a row's sum is the same whichever group forms it)
  int groups = N <= 32 ? 4 : (N <= 64 ? 2 : 1);
  while (groups > 1 && (M < groups * HG_ROWS || sizeof(float) * groups * HG_ROWS * (size_t)K > 96 * 1024)) groups >>= 1;
  const size_t smem = sizeof(float) * groups * HG_ROWS * (size_t)K;
  if (smem > 96 * 1024) return IE_BAD_SIZE;
  dim3 grid((M + groups * HG_ROWS - 1) / (groups * HG_ROWS), H);
  // few rows (decode tokens): a warp a block and 32 columns each, so that the heads' weights stream through many blocks
  int threads = HG_THREADS, z_cols = N;
  if (groups == 1 && grid.x * (size_t)H < 256 && N > 32) {
    threads = 32;
    z_cols = 32;
    grid.z = (N + 31) / 32;
  }
#define HG_GO(TX, TW, TO)                                                                                           \
  {                                                                                                                 \
    if (smem > 48 * 1024) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(heads_gemm_kernel<TX, TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                             \
      if (e != cudaSuccess) return (int)e;                                                                          \
    }                                                                                                               \
    return launch_k(heads_gemm_kernel<TX, TW, TO>, grid, threads, smem, stream, (const TX*)x, x_stride, x_head,     \
                    (const TW*)w, (TO*)out, o_stride, o_head, M, K, N, groups, z_cols);                             \
  }
  if (x_dtype == IE_F32 && w_dtype == IE_F32 && o_dtype == IE_F32) HG_GO(float, float, float);
  if (x_dtype == IE_F32 && w_dtype == IE_BF16 && o_dtype == IE_F32) HG_GO(float, bf16, float);
  if (x_dtype == IE_BF16 && w_dtype == IE_BF16 && o_dtype == IE_BF16) HG_GO(bf16, bf16, bf16);
  if (x_dtype == IE_BF16 && w_dtype == IE_F32 && o_dtype == IE_BF16) HG_GO(bf16, float, bf16);
#undef HG_GO
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ two maps of a head into one output
// maps: [n, kv groups, 2, heads in a group, hd_v] (the layout in which the two maps of a head are attention heads that
// share a key head each); out and gate: [n, heads * hd_v] with head = group * heads_in_group + head in the group.
template <typename T>
__global__ void diff_combine_kernel(const T* __restrict__ maps, int maps_stride, const T* __restrict__ gate, int gate_stride,
                                    T* __restrict__ out, int out_stride, int n_tokens, int n_heads, int rep, int hd_v,
                                    float lambda, float eps, float out_mult) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_tokens * n_heads) return;
  const int n = item / n_heads, h = item - n * n_heads;
  const int g = h / rep, hg = h - g * rep;
  const T* a1 = maps + (size_t)n * maps_stride + ((size_t)(g * 2 + 0) * rep + hg) * hd_v;
  const T* a2 = maps + (size_t)n * maps_stride + ((size_t)(g * 2 + 1) * rep + hg) * hd_v;
  float ss = 0.f;
  for (int d = lane; d < hd_v; d += 32) {
    const float o = fmaf(-lambda, to_f32(a2[d]), to_f32(a1[d]));
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  const float inv = out_mult / sqrtf(ss / (float)hd_v + eps);
  T* o_row = out + (size_t)n * out_stride + (size_t)h * hd_v;
  const T* g_row = gate != nullptr ? gate + (size_t)n * gate_stride + (size_t)h * hd_v : nullptr;
  for (int d = lane; d < hd_v; d += 32) {
    float o = fmaf(-lambda, to_f32(a2[d]), to_f32(a1[d])) * inv;
    if (g_row != nullptr) o *= 1.f / (1.f + expf(-to_f32(g_row[d])));
    o_row[d] = from_f32<T>(o);
  }
}

// bfloat16 with an even head size up to 256 and rows that start on 4 bytes: a lane takes pairs, the head stays in registers
__global__ void diff_combine_bf16_pairs_kernel(const bf16* __restrict__ maps, int maps_stride, const bf16* __restrict__ gate,
                                               int gate_stride, bf16* __restrict__ out, int out_stride, int n_tokens,
                                               int n_heads, int rep, int hd_v, float lambda, float eps, float out_mult) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_tokens * n_heads) return;
  const int n = item / n_heads, h = item - n * n_heads;
  const int g = h / rep, hg = h - g * rep;
  const bf16* a1 = maps + (size_t)n * maps_stride + ((size_t)(g * 2 + 0) * rep + hg) * hd_v;
  const bf16* a2 = maps + (size_t)n * maps_stride + ((size_t)(g * 2 + 1) * rep + hg) * hd_v;
  float2 o[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = 2 * lane + 64 * i;
    o[i] = make_float2(0.f, 0.f);
    if (d < hd_v) {
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a1 + d));
      const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a2 + d));
      o[i].x = fmaf(-lambda, y.x, x.x);
      o[i].y = fmaf(-lambda, y.y, x.y);
      ss = fmaf(o[i].x, o[i].x, ss);
      ss = fmaf(o[i].y, o[i].y, ss);
    }
  }
  ss = warp_sum(ss);
  const float inv = out_mult / sqrtf(ss / (float)hd_v + eps);
  bf16* o_row = out + (size_t)n * out_stride + (size_t)h * hd_v;
  const bf16* g_row = gate != nullptr ? gate + (size_t)n * gate_stride + (size_t)h * hd_v : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = 2 * lane + 64 * i;
    if (d < hd_v) {
      float vx = o[i].x * inv, vy = o[i].y * inv;
      if (g_row != nullptr) {
        const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g_row + d));
        vx *= 1.f / (1.f + expf(-gg.x));
        vy *= 1.f / (1.f + expf(-gg.y));
      }
      *reinterpret_cast<__nv_bfloat162*>(o_row + d) = __floats2bfloat162_rn(vx, vy);
    }
  }
}

// bfloat16 with a head of 32, 64, 128 or 256 values and rows that start on 16 bytes: a lane takes eight values, the
// hd_v / 8 lanes of a head sum their squares among themselves, a warp takes 32 / (hd_v / 8) heads
__global__ void diff_combine_bf16_vec_kernel(const bf16* __restrict__ maps, int maps_stride, const bf16* __restrict__ gate,
                                             int gate_stride, bf16* __restrict__ out, int out_stride, int n_tokens,
                                             int n_heads, int rep, int hd_v, float lambda, float eps, float out_mult) {
  pdl_trigger();
  pdl_wait();
  const int lanes = hd_v >> 3;                       // 4, 8, 16 or 32
  const int per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes, l = lane - sub * lanes;
  const long long item = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * per_warp + sub;
  const bool live = item < (long long)n_tokens * n_heads;
  const int n = live ? (int)(item / n_heads) : 0, h = live ? (int)(item - (long long)n * n_heads) : 0;
  const int g = h / rep, hg = h - g * rep;
  const int d = l * 8;
  float o[8];
  float ss = 0.f;
  {
    const uint4 x = *reinterpret_cast<const uint4*>(maps + (size_t)n * maps_stride + ((size_t)(g * 2 + 0) * rep + hg) * hd_v + d);
    const uint4 y = *reinterpret_cast<const uint4*>(maps + (size_t)n * maps_stride + ((size_t)(g * 2 + 1) * rep + hg) * hd_v + d);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
    const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 a = __bfloat1622float2(xp[t]), b = __bfloat1622float2(yp[t]);
      o[2 * t] = fmaf(-lambda, b.x, a.x);
      o[2 * t + 1] = fmaf(-lambda, b.y, a.y);
      ss = fmaf(o[2 * t], o[2 * t], ss);
      ss = fmaf(o[2 * t + 1], o[2 * t + 1], ss);
    }
  }
  for (int s = 1; s < lanes; s <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  if (!live) return;
  const float inv = out_mult / sqrtf(ss / (float)hd_v + eps);
  float gs[8];
  if (gate != nullptr) {
    const uint4 gg = *reinterpret_cast<const uint4*>(gate + (size_t)n * gate_stride + (size_t)h * hd_v + d);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gg);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 a = __bfloat1622float2(gp[t]);
      gs[2 * t] = 1.f / (1.f + expf(-a.x));
      gs[2 * t + 1] = 1.f / (1.f + expf(-a.y));
    }
  } else {
#pragma unroll
    for (int t = 0; t < 8; ++t) gs[t] = 1.f;
  }
  uint4 r;
  __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int t = 0; t < 4; ++t) rp[t] = __floats2bfloat162_rn(o[2 * t] * inv * gs[2 * t], o[2 * t + 1] * inv * gs[2 * t + 1]);
  *reinterpret_cast<uint4*>(out + (size_t)n * out_stride + (size_t)h * hd_v + d) = r;
}

extern "C" int ie_diff_combine(const void* maps, int maps_stride, const void* gate, int gate_stride, void* out,
                               int out_stride, int n_tokens, int n_heads, int n_kv_heads, int hd_v, float lambda,
                               float eps, float out_mult, int act_dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || hd_v <= 0) return IE_BAD_SIZE;
  const int rep = n_heads / n_kv_heads;
  const int warps = 8;
  const unsigned blocks = (unsigned)(((size_t)n_tokens * n_heads + warps - 1) / warps);
  if (act_dtype == IE_BF16 && (hd_v == 32 || hd_v == 64 || hd_v == 128 || hd_v == 256) && maps_stride % 8 == 0 &&
      gate_stride % 8 == 0 && out_stride % 8 == 0 && (((uintptr_t)maps | (uintptr_t)gate | (uintptr_t)out) & 15) == 0) {
    const int per_warp = 32 / (hd_v >> 3);
    const size_t n_warps = ((size_t)n_tokens * n_heads + per_warp - 1) / per_warp;
    return launch_k(diff_combine_bf16_vec_kernel, (unsigned)((n_warps + warps - 1) / warps), warps * 32, 0, stream,
                    (const bf16*)maps, maps_stride, (const bf16*)gate, gate_stride, (bf16*)out, out_stride, n_tokens, n_heads,
                    rep, hd_v, lambda, eps, out_mult);
  }
  if (act_dtype == IE_BF16 && hd_v % 2 == 0 && hd_v <= 256 && maps_stride % 2 == 0 && gate_stride % 2 == 0 && out_stride % 2 == 0 &&
      (((uintptr_t)maps | (uintptr_t)gate | (uintptr_t)out) & 3) == 0)
    return launch_k(diff_combine_bf16_pairs_kernel, blocks, warps * 32, 0, stream, (const bf16*)maps, maps_stride,
                    (const bf16*)gate, gate_stride, (bf16*)out, out_stride, n_tokens, n_heads, rep, hd_v, lambda, eps,
                    out_mult);
  if (act_dtype == IE_F32)
    return launch_k(diff_combine_kernel<float>, blocks, warps * 32, 0, stream, (const float*)maps, maps_stride,
                    (const float*)gate, gate_stride, (float*)out, out_stride, n_tokens, n_heads, rep, hd_v, lambda, eps,
                    out_mult);
  if (act_dtype == IE_BF16)
    return launch_k(diff_combine_kernel<bf16>, blocks, warps * 32, 0, stream, (const bf16*)maps, maps_stride,
                    (const bf16*)gate, gate_stride, (bf16*)out, out_stride, n_tokens, n_heads, rep, hd_v, lambda, eps,
                    out_mult);
  return IE_BAD_DTYPE;
}

IE_CHECK_API(headwise)
