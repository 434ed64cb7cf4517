// Gated linear attention with a decay per key channel, for any mix of requests in one flat batch: prompt portions
// of any length beside single decoded tokens.  Per request and head the state is a matrix S [d, dv] of 32-bit
// floats, kept in the request's state row between steps:
//
//   alpha_t = exp(logsigmoid(z_t + b) / tau)          decay per key channel, z: a 32-bit projection
//   S_t = diag(alpha_t) S_{t-1} + k_t v_t^T
//   o_t = S_t^T q_t,   q_t = q_scale * (projected query)
//
// The recurrence runs token by token, so a request's result does not depend on how its tokens were cut into steps
// or on what else is in the batch.  The parallelism is over requests, heads and the columns of S: a block owns
// (request, head, a tile of columns); a column's d rows are spread over `rs` neighbouring lanes (row r belongs to
// lane r mod rs), which meet in shuffles for the read-out.  q, k, the decays and the tile's v of a chunk of tokens
// are staged in shared memory by all threads (the decays are evaluated there, once per block), then the chunk is
// run from shared memory.
//
// State row layout (floats): S^T as [heads][dv][d].
#include "common.cuh"

#define GLA_THREADS 128
#define GLA_MAX_DIM 512
#define GLA_RPT 16  // rows of S a thread holds at most: 32 lanes x 16

__device__ __forceinline__ float gla_log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T, int RPT>
__global__ void __launch_bounds__(GLA_THREADS)
gla_recurrence_kernel(const T* __restrict__ qkv, long long row_stride, int q_off, int k_off, int v_off,
                      const float* __restrict__ z, long long z_stride, const float* __restrict__ z_bias,
                      float inv_tau, float q_scale, float* __restrict__ state, long long state_stride,
                      const int* __restrict__ cu_q, const int* __restrict__ req_slots,
                      const int* __restrict__ token_req, float* __restrict__ out, int heads, int dim, int vdim,
                      int rs, int chunk, int num_slots, int* status) {
  extern __shared__ float sm[];
  pdl_launch_dependents();
  pdl_wait();
  const int req = blockIdx.z, head = blockIdx.y;
  const int cols_per_block = GLA_THREADS / rs;
  const int tid = threadIdx.x;
  const int lane_row = tid % rs;
  const int col_in_block = tid / rs;
  const int col = blockIdx.x * cols_per_block + col_in_block;
  const bool col_ok = col < vdim;
  const int t0 = cu_q[req], t1 = cu_q[req + 1];
  if (t1 <= t0) return;
  if (token_req[t0] < 0) {  // a row that belongs to no request: zeros out, no state touched
    if (lane_row == 0 && col_ok)
      for (int t = t0; t < t1; ++t) out[((long long)t * heads + head) * vdim + col] = 0.f;
    return;
  }
  const int slot = req_slots[req];
  if (slot < 0 || slot >= num_slots) {
    if (tid == 0) ullm_report(status, ULLM_STATUS_SLOT, req, slot);
    return;
  }
  float* sq = sm;                    // [chunk][dim]
  float* sk = sq + chunk * dim;      // [chunk][dim]
  float* sa = sk + chunk * dim;      // [chunk][dim]
  float* sv = sa + chunk * dim;      // [chunk][cols_per_block]
  float* st_col = state + (long long)slot * state_stride + ((long long)head * vdim + (col_ok ? col : 0)) * dim;

  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = lane_row + i * rs;
    S[i] = (col_ok && r < dim) ? st_col[r] : 0.f;
  }
  const int col0 = blockIdx.x * cols_per_block;
  for (int c0 = t0; c0 < t1; c0 += chunk) {
    const int cn = min(chunk, t1 - c0);
    __syncthreads();  // the chunk before has been read
    for (int i = tid; i < cn * dim; i += GLA_THREADS) {
      const int t = i / dim, r = i - t * dim;
      const T* row = qkv + (long long)(c0 + t) * row_stride + head * dim + r;
      sq[i] = to_f32(row[q_off]) * q_scale;
      sk[i] = to_f32(row[k_off]);
      const float zz = z[(long long)(c0 + t) * z_stride + head * dim + r] + (z_bias != nullptr ? z_bias[head * dim + r] : 0.f);
      sa[i] = expf(gla_log_sigmoid(zz) * inv_tau);
    }
    for (int i = tid; i < cn * cols_per_block; i += GLA_THREADS) {
      const int t = i / cols_per_block, c = i - t * cols_per_block;
      sv[i] = (col0 + c < vdim) ? to_f32(qkv[(long long)(c0 + t) * row_stride + v_off + head * vdim + col0 + c]) : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < cn; ++t) {
      const float v = sv[t * cols_per_block + col_in_block];
      const float* q = sq + t * dim;
      const float* k = sk + t * dim;
      const float* a = sa + t * dim;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int r = lane_row + i * rs;
        if (r < dim) {
          S[i] = a[r] * S[i] + k[r] * v;
          acc += S[i] * q[r];
        }
      }
      for (int o = rs >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane_row == 0 && col_ok) out[((long long)(c0 + t) * heads + head) * vdim + col] = acc;
    }
  }
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int r = lane_row + i * rs;
      if (r < dim) st_col[r] = S[i];
    }
  }
}

// Lanes that share a column: as many as leave a thread about 8 rows, at most a warp.
static int gla_rs(int dim) {
  int rs = 1;
  while (rs < 32 && rs * 8 < dim) rs <<= 1;
  return rs;
}

extern "C" int ullm_gla_supported(int heads, int dim, int vdim) {
  return heads > 0 && dim > 0 && vdim > 0 && dim <= GLA_MAX_DIM;
}

extern "C" long long ullm_gla_state_floats(int heads, int dim, int vdim) { return (long long)heads * vdim * dim; }

template <typename T>
static int gla_launch(const void* qkv, long long row_stride, int q_off, int k_off, int v_off, const float* z,
                      long long z_stride, const float* z_bias, float inv_tau, float q_scale, float* state,
                      long long state_stride, const int* cu_q, const int* req_slots, const int* token_req, float* out,
                      int requests, int heads, int dim, int vdim, int num_slots, int* status, cudaStream_t st) {
  const int rs = gla_rs(dim);
  const int cpb = GLA_THREADS / rs;
  int chunk = 8192 / (3 * dim + cpb);  // at most 32 KB of shared memory
  chunk = chunk < 1 ? 1 : (chunk > 32 ? 32 : chunk);
  const size_t smem = (size_t)chunk * (3 * dim + cpb) * sizeof(float);
  const dim3 grid((vdim + cpb - 1) / cpb, heads, requests), block(GLA_THREADS);
  const int rows = (dim + rs - 1) / rs;
#define GLA_GO(RPT)                                                                                                 \
  return ullm_launch_kernel(gla_recurrence_kernel<T, RPT>, grid, block, smem, st, (const T*)qkv, row_stride, q_off,  \
                            k_off, v_off, z, z_stride, z_bias, inv_tau, q_scale, state, state_stride, cu_q, req_slots, \
                            token_req, out, heads, dim, vdim, rs, chunk, num_slots, status)
  if (rows <= 4) GLA_GO(4);
  if (rows <= 8) GLA_GO(8);
  GLA_GO(GLA_RPT);
#undef GLA_GO
}

// qkv [tokens, *]: q and k (heads x dim) and v (heads x vdim) at the given column offsets of rows `row_stride`
// apart; z [tokens, heads * dim] 32-bit (rows `z_stride` apart), `z_bias` [heads * dim] or null;
// out [tokens, heads * vdim] 32-bit.
extern "C" int ullm_gla_recurrence(int dtype, const void* qkv, long long row_stride, int q_off, int k_off, int v_off,
                                   const float* z, long long z_stride, const float* z_bias, float inv_tau,
                                   float q_scale, float* state, long long state_stride, const int* cu_q,
                                   const int* req_slots, const int* token_req, float* out, int requests, int heads,
                                   int dim, int vdim, int num_slots, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (requests < 0 || heads <= 0 || dim <= 0 || vdim <= 0 || num_slots <= 0) return ULLM_ERR_BAD_SIZE;
  if (dim > GLA_MAX_DIM || heads > 65535 || requests > 65535) return ULLM_ERR_UNSUPPORTED;
  if (state_stride < (long long)heads * vdim * dim) return ULLM_ERR_BAD_SIZE;
  if (requests == 0) return ULLM_OK;
#define GLA_ARGS                                                                                                     \
  qkv, row_stride, q_off, k_off, v_off, z, z_stride, z_bias, inv_tau, q_scale, state, state_stride, cu_q, req_slots, \
      token_req, out, requests, heads, dim, vdim, num_slots, status, st
  if (dtype == ULLM_DTYPE_F32) return gla_launch<float>(GLA_ARGS);
  if (dtype == ULLM_DTYPE_BF16) return gla_launch<__nv_bfloat16>(GLA_ARGS);
  if (dtype == ULLM_DTYPE_F16) return gla_launch<__half>(GLA_ARGS);
#undef GLA_ARGS
  return ULLM_ERR_BAD_DTYPE;
}
