// Routed feed-forward (mixture of experts) without a host round trip:
//
//   moe_route     per token: scores from the 32-bit router logits (sigmoid, or softmax over the experts), the
//                 `top` largest (ties: the lower index), their weights (the scores, optionally renormalized)
//   moe_arrange   the (token, choice) pairs grouped by expert: offsets[E + 1], sorted[p] = pair at place p,
//                 place[pair] = p
//   moe_grouped_linear   for every expert e and every place p of it:  out[p] = f(W_e . (s_p * x[row(p)]))
//                 with W_e = weights[e]; GATED: W_e stacks gate rows on up rows and
//                 out[p] = act(s_p * gate . x) * (s_p * up . x); s_p = the pair's weight when the weight
//                 multiplies the expert's input, else 1
//   moe_combine   y[t] = sum over the token's choices (in choice order) of c * rows[place], c = the weight when it
//                 multiplies the expert's output, else 1
//
// The grouped product is a tiled kernel with 32-bit accumulation for float32 and 16-bit storage alike; a block
// finds its (expert, row tile) from the offsets, so the grid depends only on the step's size.
#include "common.cuh"

#define MOE_MAX_TOP 16

__global__ void moe_route_kernel(const float* __restrict__ logits, int* __restrict__ choice, float* __restrict__ weight,
                                 int tokens, int experts, int top, int softmax_scores, int renormalize) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const float* z = logits + (long long)t * experts;
  float zmax = -INFINITY, zsum = 0.f;
  if (softmax_scores) {
    for (int e = lane; e < experts; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    for (int e = lane; e < experts; e += 32) zsum += expf(z[e] - zmax);
    zsum = warp_sum(zsum);
  }
  int taken[MOE_MAX_TOP];
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      bool used = false;
      for (int j = 0; j < k; ++j) used |= taken[j] == e;
      if (used) continue;
      const float s = softmax_scores ? expf(z[e] - zmax) / zsum : 1.f / (1.f + expf(-z[e]));
      if (s > best || (s == best && e < best_e)) {
        best = s;
        best_e = e;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    taken[k] = best_e;
    total += best;
    if (lane == 0) {
      choice[(long long)t * top + k] = best_e;
      weight[(long long)t * top + k] = best;
    }
  }
  if (renormalize && lane == 0)
    for (int k = 0; k < top; ++k) weight[(long long)t * top + k] /= total;
}

// One block.  counts in shared memory (experts <= 1024).
__global__ void moe_arrange_kernel(const int* __restrict__ choice, int pairs, int experts, int* __restrict__ offsets,
                                   int* __restrict__ sorted, int* __restrict__ place) {
  __shared__ int count[1024];
  __shared__ int cursor[1024];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = choice[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      run += count[e];
    }
    offsets[experts] = run;
  }
  __syncthreads();
  // the order inside an expert's group has no influence on any result: every place is computed by itself
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = choice[p];
    if (e >= 0 && e < experts) {
      const int at = atomicAdd(&cursor[e], 1);
      sorted[at] = p;
      place[p] = at;
    }
  }
}

#define MOE_BM 32
#define MOE_BN 64
#define MOE_BK 32
#define MOE_THREADS 256  // a thread: 2 rows x 4 columns of the tile

template <typename T, bool GATED>
__global__ void __launch_bounds__(MOE_THREADS)
moe_grouped_linear_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ weights,
                          long long expert_stride, const int* __restrict__ offsets, const int* __restrict__ sorted,
                          const float* __restrict__ pair_weight, T* __restrict__ out, int experts, int top,
                          int rows_from_pairs, int n_out, int k_dim, int act) {
  __shared__ float As[MOE_BK][MOE_BM + 1];
  __shared__ float Bs[GATED ? 2 : 1][MOE_BK][MOE_BN + 1];
  __shared__ int s_row[MOE_BM];
  __shared__ float s_scale[MOE_BM];
  pdl_launch_dependents();
  pdl_wait();
  // which expert and which tile of its rows
  int e = 0, tile = blockIdx.y, lo = 0, hi = 0;
  for (; e < experts; ++e) {
    lo = offsets[e];
    hi = offsets[e + 1];
    const int tiles = (hi - lo + MOE_BM - 1) / MOE_BM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e >= experts) return;
  const int p0 = lo + tile * MOE_BM;
  const int rows = min(MOE_BM, hi - p0);
  const int n0 = blockIdx.x * MOE_BN;
  if (threadIdx.x < MOE_BM) {
    const int i = threadIdx.x;
    int src = 0;
    float sc = 0.f;
    if (i < rows) {
      const int pair = sorted[p0 + i];
      src = rows_from_pairs ? pair / top : p0 + i;  // the token's row of x, or the place's own row
      sc = pair_weight != nullptr ? pair_weight[pair] : 1.f;
    }
    s_row[i] = src;
    s_scale[i] = sc;
  }
  __syncthreads();
  const T* W = weights + (long long)e * expert_stride;
  const int tr = threadIdx.x / 16, tc = threadIdx.x % 16;  // rows tr*2.., columns tc*4..
  float acc[GATED ? 2 : 1][2][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;

  for (int k0 = 0; k0 < k_dim; k0 += MOE_BK) {
    for (int idx = threadIdx.x; idx < MOE_BM * MOE_BK; idx += MOE_THREADS) {
      const int i = idx / MOE_BK, kk = idx % MOE_BK;
      float v = 0.f;
      if (i < rows && k0 + kk < k_dim) v = to_f32(x[(long long)s_row[i] * x_stride + k0 + kk]);
      As[kk][i] = v;
    }
    for (int idx = threadIdx.x; idx < MOE_BN * MOE_BK; idx += MOE_THREADS) {
      const int j = idx / MOE_BK, kk = idx % MOE_BK;
      const bool on = n0 + j < n_out && k0 + kk < k_dim;
      Bs[0][kk][j] = on ? to_f32(W[(long long)(n0 + j) * k_dim + k0 + kk]) : 0.f;
      if (GATED) Bs[1][kk][j] = on ? to_f32(W[(long long)(n_out + n0 + j) * k_dim + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < MOE_BK; ++kk) {
      const float a0 = As[kk][tr * 2], a1 = As[kk][tr * 2 + 1];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float b = Bs[g][kk][tc * 4 + j];
          acc[g][0][j] = fmaf(a0, b, acc[g][0][j]);
          acc[g][1][j] = fmaf(a1, b, acc[g][1][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = tr * 2 + i;
    if (r >= rows) continue;
    const float sc = s_scale[r];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tc * 4 + j;
      if (c >= n_out) continue;
      float v;
      if (GATED) {
        const float g = acc[0][i][j] * sc, u = acc[1][i][j] * sc;
        v = (act == 0 ? act_silu(g) : act_gelu_tanh(g)) * u;
      } else {
        v = acc[0][i][j] * sc;
      }
      out[(long long)(p0 + r) * n_out + c] = from_f32<T>(v);
    }
  }
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ place,
                                   const float* __restrict__ pair_weight, T* __restrict__ y, int top, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
      const long long pair = t * top + k;
      const float v = to_f32(rows[(long long)place[pair] * cols + c]);
      s += pair_weight != nullptr ? pair_weight[pair] * v : v;
    }
    y[t * cols + c] = from_f32<T>(s);
  }
}

extern "C" int ullm_moe_route(const float* logits, int* choice, float* weight, int tokens, int experts, int top,
                              int softmax_scores, int renormalize, void* stream) {
  if (tokens < 0 || experts <= 0 || top <= 0) return ULLM_ERR_BAD_SIZE;
  if (top > experts || top > MOE_MAX_TOP) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  return ullm_launch_kernel(moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, (cudaStream_t)stream, logits,
                            choice, weight, tokens, experts, top, softmax_scores, renormalize);
}

extern "C" int ullm_moe_arrange(const int* choice, int pairs, int experts, int* offsets, int* sorted, int* place,
                                void* stream) {
  if (pairs < 0 || experts <= 0) return ULLM_ERR_BAD_SIZE;
  if (experts > 1024) return ULLM_ERR_UNSUPPORTED;
  return ullm_launch_kernel(moe_arrange_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, choice, pairs, experts,
                            offsets, sorted, place);
}

template <typename T>
static int grouped_launch(const void* x, long long x_stride, const void* weights, long long expert_stride,
                          const int* offsets, const int* sorted, const float* pair_weight, void* out, int pairs,
                          int experts, int top, int rows_from_pairs, int n_out, int k_dim, int gated, int act,
                          cudaStream_t st) {
  const int row_tiles = (pairs + MOE_BM - 1) / MOE_BM + experts;  // an upper bound whatever the routing
  const dim3 grid((n_out + MOE_BN - 1) / MOE_BN, row_tiles), block(MOE_THREADS);
  if (gated)
    return ullm_launch_kernel(moe_grouped_linear_kernel<T, true>, grid, block, 0, st, (const T*)x, x_stride,
                              (const T*)weights, expert_stride, offsets, sorted, pair_weight, (T*)out, experts, top,
                              rows_from_pairs, n_out, k_dim, act);
  return ullm_launch_kernel(moe_grouped_linear_kernel<T, false>, grid, block, 0, st, (const T*)x, x_stride,
                            (const T*)weights, expert_stride, offsets, sorted, pair_weight, (T*)out, experts, top,
                            rows_from_pairs, n_out, k_dim, act);
}

// x: rows of k_dim elements (stride x_stride); row of place p = token of its pair (rows_from_pairs) or p itself.
// weights: [experts, (gated ? 2 : 1) * n_out, k_dim].  out: [pairs, n_out].
extern "C" int ullm_moe_grouped_linear(int dtype, const void* x, long long x_stride, const void* weights,
                                       long long expert_stride, const int* offsets, const int* sorted,
                                       const float* pair_weight, void* out, int pairs, int experts, int top,
                                       int rows_from_pairs, int n_out, int k_dim, int gated, int act, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (pairs < 0 || experts <= 0 || top <= 0 || n_out <= 0 || k_dim <= 0) return ULLM_ERR_BAD_SIZE;
  if (gated && act != 0 && act != 1) return ULLM_ERR_UNSUPPORTED;
  if (pairs == 0) return ULLM_OK;
  if ((pairs + MOE_BM - 1) / MOE_BM + experts > 65535) return ULLM_ERR_BAD_SIZE;
  if (dtype == ULLM_DTYPE_F32)
    return grouped_launch<float>(x, x_stride, weights, expert_stride, offsets, sorted, pair_weight, out, pairs,
                                 experts, top, rows_from_pairs, n_out, k_dim, gated, act, st);
  if (dtype == ULLM_DTYPE_BF16)
    return grouped_launch<__nv_bfloat16>(x, x_stride, weights, expert_stride, offsets, sorted, pair_weight, out,
                                         pairs, experts, top, rows_from_pairs, n_out, k_dim, gated, act, st);
  if (dtype == ULLM_DTYPE_F16)
    return grouped_launch<__half>(x, x_stride, weights, expert_stride, offsets, sorted, pair_weight, out, pairs,
                                  experts, top, rows_from_pairs, n_out, k_dim, gated, act, st);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_moe_combine(int dtype, const void* rows, const int* place, const float* pair_weight, void* y,
                                int tokens, int top, int cols, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || top <= 0 || cols <= 0) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  int threads = 32;
  while (threads < 256 && threads * 4 < cols) threads <<= 1;
  const dim3 grid(tokens), block(threads);
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(moe_combine_kernel<float>, grid, block, 0, st, (const float*)rows, place, pair_weight,
                              (float*)y, top, cols);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(moe_combine_kernel<__nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)rows,
                              place, pair_weight, (__nv_bfloat16*)y, top, cols);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(moe_combine_kernel<__half>, grid, block, 0, st, (const __half*)rows, place, pair_weight,
                              (__half*)y, top, cols);
  return ULLM_ERR_BAD_DTYPE;
}
