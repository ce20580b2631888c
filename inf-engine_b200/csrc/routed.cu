// A mixture of feed-forward experts on the device, without a trip to the host:
//   route    per token, from float32 router logits: sigmoid scores, a correction added for the choice only, the best
//            groups of neighbouring experts kept, the top experts among them, their normalised weights, and the
//            shared expert's gate; or (mode 1) the largest logits, a bias added, and the softmax over those alone;
//   sort     the (token, choice) pairs ordered by expert, and a table of row tiles, none of which spans two experts;
//   product  C[pair] = A[token of pair] W[expert of pair]^T over those tiles, optionally with silu(gate) * up in the
//            epilogue: on CUDA cores (float32 products and sums, every output one accumulator that walks k upward) for
//            the 32-bit path, on tensor cores (mma.sync, float32 accumulators) for bfloat16 operands; either way a
//            row's result does not depend on which tile or step it is in;
//   combine  out[token] = sum over its choices of weight * y[pair] + gate * shared[token], choices in order.
#include "common.cuh"

// ------------------------------------------------------------------ route
// One warp per token.  logits [n, ld]: columns 0..E-1 the experts, column `gate_col` (if >= 0) the shared expert's
// gate.  Ties go to the lower index.
template <typename TW>
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, int ld, const TW* __restrict__ correction, int* __restrict__ ids,
             float* __restrict__ weights, float* __restrict__ gate, int n_tokens, int n_experts, int top, int n_groups,
             int keep_groups, float route_scale, float weight_eps, int gate_col, int mode) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n_tokens) return;
  float* score = sm + (size_t)warp * (2 * n_experts + n_groups);   // s
  float* choice = score + n_experts;                               // s + correction, -inf once taken or shut out
  float* gscore = choice + n_experts;
  const float* z = logits + (size_t)t * ld;
  for (int e = lane; e < n_experts; e += 32) {
    const float cor = correction ? to_f32(correction[e]) : 0.f;
    // mode 1: the logits themselves (plus their bias) are both what is compared and what the weights are made of
    const float s = mode == 1 ? z[e] + cor : 1.f / (1.f + expf(-z[e]));
    score[e] = s;
    choice[e] = mode == 1 ? s : s + cor;
  }
  __syncwarp();
  const int per = n_experts / n_groups;
  if (keep_groups < n_groups) {
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;          // the two largest of the group
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > a) { b = a; a = c; } else if (c > b) b = c;
      }
      gscore[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // the groups that stay: keep_groups times the largest score left; the others are shut out afterwards
    for (int r = 0; r < keep_groups; ++r) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float c = gscore[g];
        if (c != INFINITY && (c > best || (c == best && g < at))) { best = c; at = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (lane == 0 && at != 0x7fffffff) gscore[at] = INFINITY;      // marks a kept group
      __syncwarp();
    }
    for (int e = lane; e < n_experts; e += 32)
      if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int r = 0; r < top; ++r) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float c = choice[e];
      if (c > best || (c == best && e < at && c != -INFINITY)) { best = c; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;             // nothing left to choose (scores that are not numbers): expert 0, weight as it is
    const float s = score[at];
    total += s;
    if (lane == 0) {
      ids[(size_t)t * top + r] = at;
      weights[(size_t)t * top + r] = s;
      choice[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0 && mode == 1) {
    // softmax over the chosen logits alone; the first chosen is the largest
    const float top0 = weights[(size_t)t * top];
    float sum = 0.f;
    for (int r = 0; r < top; ++r) {
      const float e = expf(weights[(size_t)t * top + r] - top0);
      weights[(size_t)t * top + r] = e;
      sum += e;
    }
    total = sum;
    weight_eps = 0.f;
  }
  if (lane == 0) {
    const float f = route_scale / (total + weight_eps);
    for (int r = 0; r < top; ++r) weights[(size_t)t * top + r] *= f;
    if (gate != nullptr) gate[t] = gate_col >= 0 ? 1.f / (1.f + expf(-z[gate_col])) : 1.f;
  }
}

extern "C" int ie_moe_route(const float* logits, int ld, const void* correction, int w_dtype, int* ids, float* weights,
                            float* gate, int n_tokens, int n_experts, int top, int n_groups, int keep_groups,
                            float route_scale, float weight_eps, int gate_col, int mode, cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (n_experts <= 0 || top <= 0 || top > n_experts || n_groups <= 0 || n_experts % n_groups || keep_groups <= 0 ||
      keep_groups > n_groups)
    return IE_BAD_SIZE;
  const size_t smem = sizeof(float) * 4 * (size_t)(2 * n_experts + n_groups);
  if (smem > 47 * 1024) return IE_BAD_SIZE;
  const unsigned blocks = (unsigned)((n_tokens + 3) / 4);
  if (w_dtype == IE_F32)
    return launch_k(route_kernel<float>, blocks, 128, smem, stream, logits, ld, (const float*)correction, ids, weights,
                    gate, n_tokens, n_experts, top, n_groups, keep_groups, route_scale, weight_eps, gate_col, mode);
  if (w_dtype == IE_BF16)
    return launch_k(route_kernel<bf16>, blocks, 128, smem, stream, logits, ld, (const bf16*)correction, ids, weights,
                    gate, n_tokens, n_experts, top, n_groups, keep_groups, route_scale, weight_eps, gate_col, mode);
  return IE_BAD_DTYPE;
}

// ------------------------------------------------------------------ sort
// One block.  sorted[pos] = pair index (token * top + choice) with the pairs of expert 0 first, then expert 1, ...;
// tiles[4 * i .. 4 * i + 3] = (expert, first position, rows, 0) for every tile of at most `tile_rows` rows; tiles
// beyond the last carry rows = 0.  The order of an expert's pairs among themselves is whatever the atomics give:
// a pair's result does not depend on its place.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int tile_rows, int* __restrict__ sorted,
                int* __restrict__ tiles, int max_tiles) {
  extern __shared__ int si[];
  int* count = si;
  int* offset = si + n_experts;
  int* cursor = si + 2 * n_experts;
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int pos = 0, nt = 0;
    for (int e = 0; e < n_experts; ++e) {
      offset[e] = pos;
      for (int r = 0; r < count[e] && nt < max_tiles; r += tile_rows, ++nt) {
        tiles[4 * nt] = e;
        tiles[4 * nt + 1] = pos + r;
        tiles[4 * nt + 2] = min(tile_rows, count[e] - r);
        tiles[4 * nt + 3] = 0;
      }
      pos += count[e];
    }
    for (; nt < max_tiles; ++nt) tiles[4 * nt] = tiles[4 * nt + 1] = tiles[4 * nt + 2] = tiles[4 * nt + 3] = 0;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < n_experts) sorted[offset[e] + atomicAdd(&cursor[e], 1)] = p;
  }
}

extern "C" int ie_moe_sort(const int* ids, int n_pairs, int n_experts, int tile_rows, int* sorted, int* tiles,
                           int max_tiles, cudaStream_t stream) {
  if (n_pairs <= 0) return IE_OK;
  if (n_experts <= 0 || tile_rows <= 0 || 3 * (size_t)n_experts * sizeof(int) > 47 * 1024) return IE_BAD_SIZE;
  return launch_k(moe_sort_kernel, 1, 1024, 3 * (size_t)n_experts * sizeof(int), stream, ids, n_pairs, n_experts,
                  tile_rows, sorted, tiles, max_tiles);
}

// ------------------------------------------------------------------ grouped product
#define MG_BM 64
#define MG_BN 64
#define MG_BK 16
#define MG_THREADS 256

// A row of tile (expert e, positions pos0 .. pos0 + rows): gather = 1: row sorted[pos] / top of A (a token's
// activations); gather = 0: row pos of A (what the product before left in sorted order).  C row: scatter = 1: row
// sorted[pos] (the pair's own place), else row pos.  W is [experts, N, K].  epi 1: columns alternate gate, up and the
// output is silu(gate) * up, N / 2 wide.
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(MG_THREADS)
moe_gemm_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, const int* __restrict__ sorted,
                const int* __restrict__ tiles, int N, int K, int lda, int ldc, long long w_expert_stride, int top,
                int gather, int scatter, int epi) {
  pdl_trigger();
  pdl_wait();
  __shared__ float As[MG_BK][MG_BM + 4];
  __shared__ float Ws[MG_BK][MG_BN + 4];
  __shared__ int a_row[MG_BM], c_row[MG_BM];
  const int tile = blockIdx.y;
  const int rows = tiles[4 * tile + 2];
  if (rows <= 0) return;
  const int expert = tiles[4 * tile], pos0 = tiles[4 * tile + 1];
  const int n0 = blockIdx.x * MG_BN;
  const int tid = threadIdx.x;
  if (tid < MG_BM) {
    int ar = -1, cr = -1;
    if (tid < rows) {
      const int pair = sorted[pos0 + tid];
      ar = gather ? pair / top : pos0 + tid;
      cr = scatter ? pair : pos0 + tid;
    }
    a_row[tid] = ar;
    c_row[tid] = cr;
  }
  __syncthreads();
  const TW* Wexp = W + (size_t)expert * w_expert_stride;
  const int tx = tid & 15, ty = tid >> 4;
  const int lr = tid >> 2, lc = (tid & 3) * 4;
  const int my_a = a_row[lr];
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += MG_BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lc + u;
      const int wn = n0 + lr;
      As[lc + u][lr] = (my_a >= 0 && k < K) ? to_f32(A[(size_t)my_a * lda + k]) : 0.f;
      Ws[lc + u][lr] = (wn < N && k < K) ? to_f32(Wexp[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MG_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int cr = c_row[ty * 4 + i];
    if (cr < 0) continue;
    if (epi == 1) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + tx * 4 + j;
        if (n + 1 < N) {
          const float g = acc[i][j];
          C[(size_t)cr * ldc + (n >> 1)] = from_f32<TC>(g / (1.f + expf(-g)) * acc[i][j + 1]);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (n < N) C[(size_t)cr * ldc + n] = from_f32<TC>(acc[i][j]);
      }
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch_moe_gemm(const void* A, const void* W, void* C, const int* sorted, const int* tiles, int max_tiles,
                           int N, int K, int lda, int ldc, long long wes, int top, int gather, int scatter, int epi,
                           cudaStream_t stream) {
  dim3 grid((N + MG_BN - 1) / MG_BN, max_tiles);
  return launch_k(moe_gemm_kernel<TA, TW, TC>, grid, MG_THREADS, 0, stream, (const TA*)A, (const TW*)W, (TC*)C, sorted,
                  tiles, N, K, lda, ldc, wes, top, gather, scatter, epi);
}

// ---- the same product on tensor cores, for bfloat16 operands (mma.sync m16n8k16, float32 accumulators): a block
// takes a tile of 64 pairs by 128 outputs and walks K in slabs of 32 through two shared-memory stages filled with
// 16-byte cp.async copies (a gathered row of A is one such stream); eight warps, two along the rows and four along
// the outputs, 32 x 32 each.  A row's sum walks k upward in the tensor core's own fixed order whatever tile the row
// lies in, so a pair's result still does not depend on its place or on the rest of the step.  K and the row strides
// must be multiples of 8 elements (16-byte copies); other shapes take the CUDA-core kernel above.
#define MM_BM 64
#define MM_BN 128
#define MM_BK 32
#define MM_LD 40          // row stride in shared memory, bfloat16 elements: 80 bytes keep ldmatrix's 8 rows on 8 bank groups
#define MM_THREADS 256

__device__ __forceinline__ uint32_t mm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mm_cp16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mm_ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TC>
__global__ void __launch_bounds__(MM_THREADS)
moe_gemm_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, TC* __restrict__ C,
                    const int* __restrict__ sorted, const int* __restrict__ tiles, int N, int K, int lda, int ldc,
                    long long w_expert_stride, int top, int gather, int scatter, int epi) {
  pdl_trigger();
  pdl_wait();
  __shared__ __align__(16) bf16 As[2][MM_BM * MM_LD];
  __shared__ __align__(16) bf16 Ws[2][MM_BN * MM_LD];
  __shared__ int a_row[MM_BM], c_row[MM_BM];
  const int tile = blockIdx.y;
  const int rows = tiles[4 * tile + 2];
  if (rows <= 0) return;
  const int expert = tiles[4 * tile], pos0 = tiles[4 * tile + 1];
  const int n0 = blockIdx.x * MM_BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < MM_BM) {
    int ar = -1, cr = -1;
    if (tid < rows) {
      const int pair = sorted[pos0 + tid];
      ar = gather ? pair / top : pos0 + tid;
      cr = scatter ? pair : pos0 + tid;
    }
    a_row[tid] = ar;
    c_row[tid] = cr;
  }
  __syncthreads();
  const bf16* Wexp = W + (size_t)expert * w_expert_stride;
  const int lrow = tid >> 2, lch = (tid & 3) * 8;          // this thread's row and 8-element chunk of a slab
  const int my_a = a_row[lrow];
  auto load_stage = [&](int s, int k0) {
    const int k = k0 + lch;
    const bool kin = k < K;
    mm_cp16(mm_smem(&As[s][lrow * MM_LD + lch]), (my_a >= 0 && kin) ? (const void*)(A + (size_t)my_a * lda + k) : (const void*)A,
            (my_a >= 0 && kin) ? 16 : 0);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int wr = lrow + 64 * u, wn = n0 + wr;
      mm_cp16(mm_smem(&Ws[s][wr * MM_LD + lch]), (wn < N && kin) ? (const void*)(Wexp + (size_t)wn * K + k) : (const void*)W,
              (wn < N && kin) ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int wm = warp & 1, wn = warp >> 1;                   // 2 x 4 warps, 32 x 32 outputs each
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
  const int nk = (K + MM_BK - 1) / MM_BK;
  load_stage(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    const int s = kt & 1;
    if (kt + 1 < nk) {
      load_stage(s ^ 1, (kt + 1) * MM_BK);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < MM_BK; ks += 16) {
      uint32_t af[2][4], bfr[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        mm_ldsm4(af[mt], mm_smem(&As[s][(wm * 32 + mt * 16 + (lane & 15)) * MM_LD + ks + (lane >> 4) * 8]));
#pragma unroll
      for (int np = 0; np < 2; ++np)
        mm_ldsm4(bfr[np], mm_smem(&Ws[s][(wn * 32 + np * 16 + (lane & 7) + (lane >> 4) * 8) * MM_LD + ks + ((lane >> 3) & 1) * 8]));
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mm_mma(acc[mt][nt], af[mt], bfr[nt >> 1][(nt & 1) * 2], bfr[nt >> 1][(nt & 1) * 2 + 1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int cr = c_row[wm * 32 + mt * 16 + (lane >> 2) + half * 8];
      if (cr < 0) continue;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int n = n0 + wn * 32 + nt * 8 + (lane & 3) * 2;
        const float x0 = acc[mt][nt][half * 2], x1 = acc[mt][nt][half * 2 + 1];
        if (epi == 1) {
          if (n + 1 < N) C[(size_t)cr * ldc + (n >> 1)] = from_f32<TC>(x0 / (1.f + expf(-x0)) * x1);
        } else {
          if (n < N) C[(size_t)cr * ldc + n] = from_f32<TC>(x0);
          if (n + 1 < N) C[(size_t)cr * ldc + n + 1] = from_f32<TC>(x1);
        }
      }
    }
  }
}

extern "C" int ie_moe_tile_rows() { return MG_BM; }

extern "C" int ie_moe_gemm(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                           const int* sorted, const int* tiles, int max_tiles, int N, int K, int lda, int ldc,
                           long long w_expert_stride, int top, int gather, int scatter, int epi, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return IE_OK;
  if (K <= 0 || top <= 0 || (epi == 1 && (N & 1))) return IE_BAD_SIZE;
  if (a_dtype == IE_BF16 && w_dtype == IE_BF16 && K % 8 == 0 && lda % 8 == 0 && w_expert_stride % 8 == 0 &&
      (((uintptr_t)A | (uintptr_t)W) & 15) == 0) {
    static_assert(MM_BM == MG_BM, "both kernels walk the same tiles");
    dim3 grid((N + MM_BN - 1) / MM_BN, max_tiles);
    if (c_dtype == IE_BF16)
      return launch_k(moe_gemm_mma_kernel<bf16>, grid, MM_THREADS, 0, stream, (const bf16*)A, (const bf16*)W, (bf16*)C,
                      sorted, tiles, N, K, lda, ldc, w_expert_stride, top, gather, scatter, epi);
    return launch_k(moe_gemm_mma_kernel<float>, grid, MM_THREADS, 0, stream, (const bf16*)A, (const bf16*)W, (float*)C,
                    sorted, tiles, N, K, lda, ldc, w_expert_stride, top, gather, scatter, epi);
  }
  const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
#define MG_GO(TA, TW, TC)                                                                                         \
  return launch_moe_gemm<TA, TW, TC>(A, W, C, sorted, tiles, max_tiles, N, K, lda, ldc, w_expert_stride, top, gather, \
                                     scatter, epi, stream)
  switch (code) {
    case 0: MG_GO(float, float, float);
    case 2: MG_GO(float, bf16, float);
    case 4: MG_GO(bf16, float, float);
    case 5: MG_GO(bf16, float, bf16);
    case 6: MG_GO(bf16, bf16, float);
    case 7: MG_GO(bf16, bf16, bf16);
    default: return IE_BAD_DTYPE;
  }
#undef MG_GO
}

// ------------------------------------------------------------------ combine
// out[t, :] = sum_r weights[t, r] * y[t * top + r, :]  (r upward)  + gate[t] * shared[t, :]
template <typename TS>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights,
                                   const float* __restrict__ gate, const TS* __restrict__ shared_out, int shared_stride,
                                   float* __restrict__ out, int d, int top) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float* w = weights + (size_t)t * top;
  const float g = (gate != nullptr && shared_out != nullptr) ? gate[t] : 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < top; ++r) acc = fmaf(w[r], y[((size_t)t * top + r) * d + i], acc);
    if (shared_out != nullptr) acc = fmaf(g, to_f32(shared_out[(size_t)t * shared_stride + i]), acc);
    out[(size_t)t * d + i] = acc;
  }
}

extern "C" int ie_moe_combine(const float* y, const float* weights, const float* gate, const void* shared_out,
                              int shared_dtype, int shared_stride, float* out, int n_tokens, int d, int top,
                              cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  const int threads = d >= 1024 ? 256 : 128;
  if (shared_out == nullptr || shared_dtype == IE_F32)
    return launch_k(moe_combine_kernel<float>, n_tokens, threads, 0, stream, y, weights, gate,
                    (const float*)shared_out, shared_stride, out, d, top);
  if (shared_dtype == IE_BF16)
    return launch_k(moe_combine_kernel<bf16>, n_tokens, threads, 0, stream, y, weights, gate, (const bf16*)shared_out,
                    shared_stride, out, d, top);
  return IE_BAD_DTYPE;
}
