// Heads of an attention layer whose softmax weights are mixed across heads, before and after the attention itself.
//
// qkv_prepare: per token, for the three projections q, k and v of one row buffer each:
//   * an optional bias of the row's size is added;
//   * every head (q: q_heads of hd, k: k_heads of hd, v: v_heads of hd_v) is divided by its root mean square
//     (x / sqrt(mean(x^2) + eps), no gain) when the side's flag says so: float32 sums and quotients;
//   * q is written back in place; k goes to its page slot of a pool [page, k_heads, page_size, hd]; v to a pool
//     [page, pool_v_heads, page_size, v_heads * hd_v / pool_v_heads]: with pool_v_heads = 1 all value heads of a token
//     lie side by side in one row, which is what an attention that applies a head's weights to EVERY value head reads.
//   A token whose slot is negative (padding) writes nothing to the pools.
//
// talk_combine: with A[n, g, c, :] = (softmax weights of query head g) applied to the values of value head c, and T the
//   [heads, heads] matrix that mixes the weights of the heads,
//       out[n, h, :] = sum_g T[h, g] * A[n, g, c(h), :] * sigmoid(gate[n, h, :]),   c(h) = h / (heads / value heads):
//   mixing the weights and then applying them to a head's own values is this sum of the unmixed heads' results.  The
//   value heads may arrive in slices (`a` then holds the value heads c0 .. c0 + nc - 1 only, and the launch writes the
//   output heads that read those).
//   float32 sums, in ascending g.
#include "common.cuh"

struct PrepSide {
  void* x;            // [n, heads * hd] rows, row stride `stride`
  const void* bias;   // [heads * hd] or null
  int stride, heads, hd, norm;
};

template <typename TA, typename TW>
__global__ void qkv_prepare_kernel(PrepSide qs, PrepSide ks, PrepSide vs, float eps,
                                   const int* __restrict__ slot_mapping, TA* __restrict__ kpool, TA* __restrict__ vpool,
                                   int pool_v_heads, int page_size) {
  extern __shared__ float rows[];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const PrepSide sides[3] = {qs, ks, vs};
  int off[4];
  off[0] = 0;
  for (int s = 0; s < 3; ++s) off[s + 1] = off[s] + sides[s].heads * sides[s].hd;
  for (int s = 0; s < 3; ++s) {
    const PrepSide& sd = sides[s];
    const TA* xr = (const TA*)sd.x + (size_t)n * sd.stride;
    const TW* b = (const TW*)sd.bias;
    const int w = sd.heads * sd.hd;
    for (int i = threadIdx.x; i < w; i += blockDim.x) rows[off[s] + i] = to_f32(xr[i]) + (b ? to_f32(b[i]) : 0.f);
  }
  __syncthreads();
  // norms: a warp a head, the three sides' heads in one list
  const int total_heads = qs.heads + ks.heads + vs.heads;
  for (int hh = warp; hh < total_heads; hh += n_warps) {
    const int s = hh < qs.heads ? 0 : (hh < qs.heads + ks.heads ? 1 : 2);
    const PrepSide& sd = sides[s];
    if (!sd.norm) continue;
    const int h = hh - (s == 0 ? 0 : (s == 1 ? qs.heads : qs.heads + ks.heads));
    float* hx = rows + off[s] + h * sd.hd;
    float ss = 0.f;
    for (int d = lane; d < sd.hd; d += 32) ss = fmaf(hx[d], hx[d], ss);
    ss = warp_sum(ss);
    const float r = sqrtf(ss / (float)sd.hd + eps);
    for (int d = lane; d < sd.hd; d += 32) hx[d] = hx[d] / r;
  }
  __syncthreads();
  const int slot = slot_mapping ? IE_SLOT(slot_mapping[n]) : -1;
  const int page = slot >= 0 ? slot / page_size : 0, at = slot >= 0 ? slot % page_size : 0;
  TA* qr = (TA*)qs.x + (size_t)n * qs.stride;
  for (int i = threadIdx.x; i < off[1]; i += blockDim.x) qr[i] = from_f32<TA>(rows[i]);
  if (slot < 0) return;
  if (kpool != nullptr) {
    const int w = ks.heads * ks.hd;
    for (int i = threadIdx.x; i < w; i += blockDim.x) {
      const int h = i / ks.hd, le = i - h * ks.hd;
      kpool[(((size_t)page * ks.heads + h) * page_size + at) * ks.hd + le] = from_f32<TA>(rows[off[1] + i]);
    }
  }
  if (vpool != nullptr) {
    const int w = vs.heads * vs.hd, pw = w / pool_v_heads;
    for (int i = threadIdx.x; i < w; i += blockDim.x) {
      const int h = i / pw, le = i - h * pw;
      vpool[(((size_t)page * pool_v_heads + h) * page_size + at) * pw + le] = from_f32<TA>(rows[off[2] + i]);
    }
  }
}

extern "C" int ie_qkv_prepare(void* q, int q_stride, int q_heads, const void* q_bias, int q_norm, void* k, int k_stride,
                              int k_heads, const void* k_bias, int k_norm, int hd, void* v, int v_stride, int v_heads,
                              int hd_v, const void* v_bias, int v_norm, int w_dtype, float eps, const int* slot_mapping,
                              void* kpool, void* vpool, int pool_v_heads, int n_tokens, int page_size, int act_dtype,
                              cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (q_heads <= 0 || k_heads <= 0 || v_heads <= 0 || hd <= 0 || hd_v <= 0 || page_size <= 0) return IE_BAD_SIZE;
  if (pool_v_heads <= 0 || v_heads % pool_v_heads) return IE_BAD_SIZE;
  PrepSide qs{q, q_bias, q_stride, q_heads, hd, q_norm};
  PrepSide ks{k, k_bias, k_stride, k_heads, hd, k_norm};
  PrepSide vs{v, v_bias, v_stride, v_heads, hd_v, v_norm};
  const size_t smem = sizeof(float) * ((size_t)(q_heads + k_heads) * hd + (size_t)v_heads * hd_v);
  if (smem > 200 * 1024) return IE_BAD_SIZE;
#define QP_GO(TA, TW)                                                                                              \
  {                                                                                                                \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(qkv_prepare_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                            \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    return launch_k(qkv_prepare_kernel<TA, TW>, n_tokens, 256, smem, stream, qs, ks, vs, eps, slot_mapping,        \
                    (TA*)kpool, (TA*)vpool, pool_v_heads, page_size);                                              \
  }
  if (act_dtype == IE_F32 && w_dtype == IE_F32) QP_GO(float, float);
  if (act_dtype == IE_F32 && w_dtype == IE_BF16) QP_GO(float, bf16);
  if (act_dtype == IE_BF16 && w_dtype == IE_F32) QP_GO(bf16, float);
  if (act_dtype == IE_BF16 && w_dtype == IE_BF16) QP_GO(bf16, bf16);
#undef QP_GO
  return IE_BAD_DTYPE;
}

// A block a token; thread j walks the output coordinates (h, d).  `a` is [n, heads, nc * hd_v] (the slice's value heads
// side by side), `talk` float32 [heads, heads] in shared memory.
template <typename TA>
__global__ void talk_combine_kernel(const TA* __restrict__ a, int a_stride, const float* __restrict__ talk,
                                    const TA* __restrict__ gate, int gate_stride, TA* __restrict__ out, int out_stride,
                                    int heads, int v_heads, int hd_v, int c0, int nc) {
  extern __shared__ float ts[];
  pdl_trigger();
  for (int i = threadIdx.x; i < heads * heads; i += blockDim.x) ts[i] = talk[i];
  pdl_wait();
  __syncthreads();
  const int n = blockIdx.x;
  const int rep = heads / v_heads, slice_w = nc * hd_v;
  const TA* an = a + (size_t)n * a_stride;
  for (int i = threadIdx.x; i < rep * slice_w; i += blockDim.x) {
    // coordinate i of the slice's share of the output: value head c0 + i / (rep * hd_v), then head in group, then d
    const int cl = i / (rep * hd_v), rem = i - cl * rep * hd_v;
    const int h = (c0 + cl) * rep + rem / hd_v, d = rem % hd_v;
    float acc = 0.f;
    const float* trow = ts + h * heads;
    for (int g = 0; g < heads; ++g) acc = fmaf(trow[g], to_f32(an[(size_t)g * slice_w + cl * hd_v + d]), acc);
    const int col = h * hd_v + d;
    if (gate != nullptr) acc = acc / (1.f + expf(-to_f32(gate[(size_t)n * gate_stride + col])));
    out[(size_t)n * out_stride + col] = from_f32<TA>(acc);
  }
}

// bfloat16 rows in 16-byte pieces: a thread forms eight neighbouring coordinates of one head's output
__global__ void talk_combine_vec_kernel(const bf16* __restrict__ a, int a_stride, const float* __restrict__ talk,
                                        const bf16* __restrict__ gate, int gate_stride, bf16* __restrict__ out,
                                        int out_stride, int heads, int v_heads, int hd_v, int c0, int nc) {
  extern __shared__ float ts[];
  pdl_trigger();
  for (int i = threadIdx.x; i < heads * heads; i += blockDim.x) ts[i] = talk[i];
  pdl_wait();
  __syncthreads();
  const int n = blockIdx.x;
  const int rep = heads / v_heads, slice_w = nc * hd_v, per_head = hd_v >> 3;
  const bf16* an = a + (size_t)n * a_stride;
  for (int i = threadIdx.x; i < nc * rep * per_head; i += blockDim.x) {
    const int cl = i / (rep * per_head), rem = i - cl * rep * per_head;
    const int h = (c0 + cl) * rep + rem / per_head, d = (rem % per_head) << 3;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const float* trow = ts + h * heads;
    const bf16* src = an + cl * hd_v + d;
#pragma unroll 4
    for (int g = 0; g < heads; ++g) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + (size_t)g * slice_w);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float w = trow[g];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p2[j]);
        acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
      }
    }
    const int col = h * hd_v + d;
    if (gate != nullptr) {
      const uint4 gr = *reinterpret_cast<const uint4*>(gate + (size_t)n * gate_stride + col);
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gr);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(gp[j]);
        acc[2 * j] = acc[2 * j] / (1.f + expf(-f.x));
        acc[2 * j + 1] = acc[2 * j + 1] / (1.f + expf(-f.y));
      }
    }
    uint4 res;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
    for (int j = 0; j < 4; ++j) rp[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)n * out_stride + col) = res;
  }
}

extern "C" int ie_talk_combine(const void* a, int a_stride, const float* talk, const void* gate, int gate_stride,
                               void* out, int out_stride, int n, int heads, int v_heads, int hd_v, int c0, int nc,
                               int act_dtype, cudaStream_t stream) {
  if (n <= 0) return IE_OK;
  if (heads <= 0 || v_heads <= 0 || heads % v_heads || hd_v <= 0 || c0 < 0 || nc <= 0 || c0 + nc > v_heads)
    return IE_BAD_SIZE;
  const size_t smem = sizeof(float) * (size_t)heads * heads;
  if (smem > 48 * 1024) return IE_BAD_SIZE;
  if (act_dtype == IE_BF16 && (hd_v & 7) == 0 && (a_stride & 7) == 0 && (out_stride & 7) == 0 &&
      ((((uintptr_t)a) | ((uintptr_t)out)) & 15) == 0 &&
      (gate == nullptr || ((gate_stride & 7) == 0 && (((uintptr_t)gate) & 15) == 0))) {
    const int work = nc * (heads / v_heads) * (hd_v >> 3);
    const int threads = work >= 256 ? 256 : ((work + 31) / 32) * 32;
    return launch_k(talk_combine_vec_kernel, n, threads, smem, stream, (const bf16*)a, a_stride, talk, (const bf16*)gate,
                    gate_stride, (bf16*)out, out_stride, heads, v_heads, hd_v, c0, nc);
  }
  if (act_dtype == IE_F32)
    return launch_k(talk_combine_kernel<float>, n, 256, smem, stream, (const float*)a, a_stride, talk,
                    (const float*)gate, gate_stride, (float*)out, out_stride, heads, v_heads, hd_v, c0, nc);
  if (act_dtype == IE_BF16)
    return launch_k(talk_combine_kernel<bf16>, n, 256, smem, stream, (const bf16*)a, a_stride, talk, (const bf16*)gate,
                    gate_stride, (bf16*)out, out_stride, heads, v_heads, hd_v, c0, nc);
  return IE_BAD_DTYPE;
}

IE_CHECK_API(headmix)
