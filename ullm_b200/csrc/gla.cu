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
// (request, head, a tile of columns); a column's d rows are spread over `rs` neighbouring lanes in pieces of four
// (rows 4 (g rs + lane) .. + 3 belong to that lane: one 16-byte read of shared memory per piece and operand, free
// of bank conflicts), which meet in shuffles for the read-out.  A first kernel turns the decay's projection into the
// decays (once per token and channel); q, k, the decays and the tile's v of a chunk of tokens are staged in shared
// memory by a second set of threads of the block while the first set runs the chunk before (two buffers).
//
// State row layout (floats): S^T as [heads][dv][d].
#include "common.cuh"

#include <type_traits>

#define GLA_THREADS 128    // threads that run the recurrence; as many again stage the next chunk
#define GLA_MAX_DIM 512
#define GLA_RPT 16         // rows of S a thread holds at most: 32 lanes x 16

__device__ __forceinline__ float gla_log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// z (32-bit, rows `stride` apart) <- exp(logsigmoid(z + bias) / tau) in place: the decays, evaluated once per
// token and channel in front of the recurrence, whose blocks would otherwise each evaluate them again.
__global__ void gla_decay_kernel(float* __restrict__ z, long long stride, const float* __restrict__ bias, int cols,
                                 long long total, float inv_tau) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / cols;
  const int c = (int)(i - t * cols);
  float* p = z + t * stride + c;
  *p = expf(gla_log_sigmoid(*p + (bias != nullptr ? bias[c] : 0.f)) * inv_tau);
}

// Threads 0 .. 127 run the recurrence on the chunk of tokens that lies in one half of shared memory while threads
// 128 .. 255 stage the next chunk (q scaled, k, the decays, the tile's v; 32-bit) in the other half.  A staged row
// is padded to RPT * rs entries with q = k = decay = 0, so the row loop has no bounds checks: the padded rows of S
// stay zero.  CPT: neighbouring value columns a thread holds; the q, k and decay it reads serve all of them.
template <typename T, int RPT, int CPT>
__global__ void __launch_bounds__(2 * GLA_THREADS)
gla_recurrence_kernel(const T* __restrict__ qkv, long long row_stride, int q_off, int k_off, int v_off,
                      const float* __restrict__ decay, long long decay_stride, float q_scale,
                      float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                      const int* __restrict__ req_slots, const int* __restrict__ token_req, float* __restrict__ out,
                      int heads, int dim, int vdim, int rs, int chunk, int num_slots, int* status) {
  extern __shared__ __align__(16) float sm[];
  pdl_launch_dependents();
  pdl_wait();
  const int req = blockIdx.z, head = blockIdx.y;
  const int groups = GLA_THREADS / rs;       // column groups of a block
  const int cols_per_block = groups * CPT;
  const bool loader = threadIdx.x >= GLA_THREADS;
  const int tid = threadIdx.x & (GLA_THREADS - 1);
  const int lane_row = tid % rs;
  const int group = tid / rs;
  const int col0 = blockIdx.x * cols_per_block;
  const int col = col0 + group * CPT;        // the thread's first column
  const int dimp = RPT * rs;                 // a staged row, padded
  const int t0 = cu_q[req], t1 = cu_q[req + 1];
  if (t1 <= t0) return;
  if (token_req[t0] < 0) {  // a row that belongs to no request: zeros out, no state touched
    if (!loader && lane_row == 0)
      for (int t = t0; t < t1; ++t)
        for (int c = 0; c < CPT; ++c)
          if (col + c < vdim) out[((long long)t * heads + head) * vdim + col + c] = 0.f;
    return;
  }
  const int slot = req_slots[req];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) ullm_report(status, ULLM_STATUS_SLOT, req, slot);
    return;
  }
  const int buf_floats = chunk * (3 * dimp + cols_per_block);
  const bool vec8 = std::is_same<T, __nv_bfloat16>::value && (dim & 7) == 0 && (dimp & 7) == 0 && (q_off & 7) == 0 &&
                    (k_off & 7) == 0 && (row_stride & 7) == 0 && (decay_stride & 3) == 0 &&
                    (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 && (reinterpret_cast<uintptr_t>(decay) & 15) == 0;
  float* st_head = state + (long long)slot * state_stride + (long long)head * vdim * dim;

  auto fill = [&](int which, int c0, int cn) {  // loader threads: tokens c0 .. c0 + cn - 1 into buffer `which`
    float* sq = sm + which * buf_floats;  // [chunk][dimp]
    float* sk = sq + chunk * dimp;
    float* sa = sk + chunk * dimp;
    float* sv = sa + chunk * dimp;        // [chunk][cols_per_block]
    if (vec8) {
      // bfloat16 rows that allow 16-byte pieces: a thread moves 8 neighbouring entries of q, k and the decays per
      // item, two items in flight
      const int per_tok = dimp >> 3, n8 = cn * per_tok;
      for (int g0 = tid; g0 < n8; g0 += 2 * GLA_THREADS) {
        uint4 rq[2], rk[2];
        float4 ra[2][2];
        bool live[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int g = g0 + j * GLA_THREADS;
          live[j] = false;
          if (g < n8) {
            const int t = g / per_tok, r = (g - t * per_tok) << 3;
            if (r < dim) {
              live[j] = true;
              const T* row = qkv + (long long)(c0 + t) * row_stride + head * dim + r;
              rq[j] = *reinterpret_cast<const uint4*>(row + q_off);
              rk[j] = *reinterpret_cast<const uint4*>(row + k_off);
              const float4* ap = reinterpret_cast<const float4*>(decay + (long long)(c0 + t) * decay_stride + head * dim + r);
              ra[j][0] = ap[0];
              ra[j][1] = ap[1];
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int g = g0 + j * GLA_THREADS;
          if (g < n8) {
            const int i = g << 3;
            float4 a, b, c, d;
            a = b = c = d = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live[j]) {
              const __nv_bfloat16* eq = reinterpret_cast<const __nv_bfloat16*>(&rq[j]);
              const __nv_bfloat16* ek = reinterpret_cast<const __nv_bfloat16*>(&rk[j]);
              a = make_float4(__bfloat162float(eq[0]) * q_scale, __bfloat162float(eq[1]) * q_scale,
                              __bfloat162float(eq[2]) * q_scale, __bfloat162float(eq[3]) * q_scale);
              b = make_float4(__bfloat162float(eq[4]) * q_scale, __bfloat162float(eq[5]) * q_scale,
                              __bfloat162float(eq[6]) * q_scale, __bfloat162float(eq[7]) * q_scale);
              c = make_float4(__bfloat162float(ek[0]), __bfloat162float(ek[1]), __bfloat162float(ek[2]), __bfloat162float(ek[3]));
              d = make_float4(__bfloat162float(ek[4]), __bfloat162float(ek[5]), __bfloat162float(ek[6]), __bfloat162float(ek[7]));
            }
            *reinterpret_cast<float4*>(sq + i) = a;
            *reinterpret_cast<float4*>(sq + i + 4) = b;
            *reinterpret_cast<float4*>(sk + i) = c;
            *reinterpret_cast<float4*>(sk + i + 4) = d;
            *reinterpret_cast<float4*>(sa + i) = live[j] ? ra[j][0] : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(sa + i + 4) = live[j] ? ra[j][1] : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
      }
    } else
    for (int i = tid; i < cn * dimp; i += GLA_THREADS) {
      const int t = i / dimp, r = i - t * dimp;
      float qv = 0.f, kv = 0.f, av = 0.f;
      if (r < dim) {
        const T* row = qkv + (long long)(c0 + t) * row_stride + head * dim + r;
        qv = to_f32(row[q_off]) * q_scale;
        kv = to_f32(row[k_off]);
        av = decay[(long long)(c0 + t) * decay_stride + head * dim + r];
      }
      sq[i] = qv;
      sk[i] = kv;
      sa[i] = av;
    }
    for (int i = tid; i < cn * cols_per_block; i += GLA_THREADS) {
      const int t = i / cols_per_block, c = i - t * cols_per_block;
      sv[i] = (col0 + c < vdim) ? to_f32(qkv[(long long)(c0 + t) * row_stride + v_off + head * vdim + col0 + c]) : 0.f;
    }
  };

  float S[RPT][CPT];
  if (!loader) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int r = ((i >> 2) * rs + lane_row) * 4 + (i & 3);
#pragma unroll
      for (int c = 0; c < CPT; ++c) S[i][c] = (col + c < vdim && r < dim) ? st_head[(long long)(col + c) * dim + r] : 0.f;
    }
  } else {
    fill(0, t0, min(chunk, t1 - t0));
  }
  __syncthreads();
  int which = 0;
  for (int c0 = t0; c0 < t1; c0 += chunk, which ^= 1) {
    const int cn = min(chunk, t1 - c0);
    if (loader) {
      if (c0 + chunk < t1) fill(which ^ 1, c0 + chunk, min(chunk, t1 - c0 - chunk));
    } else {
      const float* sq = sm + which * buf_floats;
      const float* sk = sq + chunk * dimp;
      const float* sa = sk + chunk * dimp;
      const float* sv = sa + chunk * dimp;
      // Four tokens at a time: only S carries a dependence from token to token (one multiply-add per row); the
      // read-outs of the four tokens are summed over the lanes together, so that a warp waits for one chain of
      // shuffles per four tokens instead of one per token.
      constexpr int TB = 4;
      for (int t = 0; t < cn; t += TB) {
        float acc[TB][CPT];
#pragma unroll
        for (int j = 0; j < TB; ++j) {
#pragma unroll
          for (int c = 0; c < CPT; ++c) acc[j][c] = 0.f;
          if (t + j < cn) {
            float v[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) v[c] = sv[(t + j) * cols_per_block + group * CPT + c];
            const float4* q4 = reinterpret_cast<const float4*>(sq + (t + j) * dimp) + lane_row;
            const float4* k4 = reinterpret_cast<const float4*>(sk + (t + j) * dimp) + lane_row;
            const float4* a4 = reinterpret_cast<const float4*>(sa + (t + j) * dimp) + lane_row;
#pragma unroll
            for (int g = 0; g < RPT / 4; ++g) {
              const float4 av = a4[g * rs], kv = k4[g * rs], qv = q4[g * rs];
              const float ar[4] = {av.x, av.y, av.z, av.w}, kr[4] = {kv.x, kv.y, kv.z, kv.w},
                          qr[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                  S[4 * g + e][c] = fmaf(ar[e], S[4 * g + e][c], kr[e] * v[c]);
                  acc[j][c] = fmaf(S[4 * g + e][c], qr[e], acc[j][c]);
                }
              }
            }
          }
        }
        for (int o = rs >> 1; o > 0; o >>= 1) {
#pragma unroll
          for (int j = 0; j < TB; ++j)
#pragma unroll
            for (int c = 0; c < CPT; ++c) acc[j][c] += __shfl_xor_sync(0xffffffffu, acc[j][c], o);
        }
        if (lane_row == 0) {
#pragma unroll
          for (int j = 0; j < TB; ++j)
            if (t + j < cn) {
#pragma unroll
              for (int c = 0; c < CPT; ++c)
                if (col + c < vdim) out[((long long)(c0 + t + j) * heads + head) * vdim + col + c] = acc[j][c];
            }
        }
      }
    }
    __syncthreads();  // the next chunk is staged, this one has been read
  }
  if (!loader) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int r = ((i >> 2) * rs + lane_row) * 4 + (i & 3);
#pragma unroll
      for (int c = 0; c < CPT; ++c)
        if (col + c < vdim && r < dim) st_head[(long long)(col + c) * dim + r] = S[i][c];
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
static int gla_launch(const void* qkv, long long row_stride, int q_off, int k_off, int v_off, float* z,
                      long long z_stride, const float* z_bias, float inv_tau, float q_scale, float* state,
                      long long state_stride, const int* cu_q, const int* req_slots, const int* token_req, float* out,
                      int tokens, int requests, int heads, int dim, int vdim, int num_slots, int* status, cudaStream_t st) {
  const long long total = (long long)tokens * heads * dim;
  if (total > 0) {
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
    const int rc = ullm_launch_kernel(gla_decay_kernel, dim3((int)blocks), dim3(256), 0, st, z, z_stride, z_bias,
                                      heads * dim, total, inv_tau);
    if (rc != ULLM_OK) return rc;
  }
  const int rs = gla_rs(dim);
  const int groups = GLA_THREADS / rs;
  const int rows = (dim + rs - 1) / rs;
  const int rpt = rows <= 4 ? 4 : (rows <= 8 ? 8 : GLA_RPT);
  // Columns per thread (1, 2 or 4): the recurrence is a chain per token, so the time is (waves of blocks) x (a
  // token's cost, which grows slowly with the columns a thread holds); two blocks are resident per SM.
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int cpt = 1;
  if (rpt <= 8) {
    double best = 1e30;
    for (int c = 1; c <= 4; c *= 2) {
      const long long blocks = (long long)((vdim + c * groups - 1) / (c * groups)) * heads * requests;
      const double cost = (double)((blocks + 2LL * sms - 1) / (2LL * sms)) * (1.0 + 0.25 * (c - 1));
      if (cost < best - 1e-9) {
        best = cost;
        cpt = c;
      }
    }
  }
  const int cpb = groups * cpt;
  const int dimp = rpt * rs;
  int chunk = (40 * 1024 / 4) / (2 * (3 * dimp + cpb));  // two buffers in at most 40 KB of shared memory
  chunk = chunk < 1 ? 1 : (chunk > 32 ? 32 : chunk);
  const size_t smem = (size_t)2 * chunk * (3 * dimp + cpb) * sizeof(float);
  const dim3 grid((vdim + cpb - 1) / cpb, heads, requests), block(2 * GLA_THREADS);
#define GLA_GO(RPT, CPT)                                                                                              \
  return ullm_launch_kernel(gla_recurrence_kernel<T, RPT, CPT>, grid, block, smem, st, (const T*)qkv, row_stride,      \
                            q_off, k_off, v_off, (const float*)z, z_stride, q_scale, state, state_stride, cu_q,        \
                            req_slots, token_req, out, heads, dim, vdim, rs, chunk, num_slots, status)
  if (rpt == 4) {
    if (cpt == 4) GLA_GO(4, 4);
    if (cpt == 2) GLA_GO(4, 2);
    GLA_GO(4, 1);
  }
  if (rpt == 8) {
    if (cpt == 4) GLA_GO(8, 4);
    if (cpt == 2) GLA_GO(8, 2);
    GLA_GO(8, 1);
  }
  GLA_GO(GLA_RPT, 1);
#undef GLA_GO
}

// qkv [tokens, *]: q and k (heads x dim) and v (heads x vdim) at the given column offsets of rows `row_stride`
// apart; z [tokens, heads * dim] 32-bit (rows `z_stride` apart), `z_bias` [heads * dim] or null: the decay's
// projection, REPLACED by the decays; out [tokens, heads * vdim] 32-bit.
extern "C" int ullm_gla_recurrence(int dtype, const void* qkv, long long row_stride, int q_off, int k_off, int v_off,
                                   float* z, long long z_stride, const float* z_bias, float inv_tau,
                                   float q_scale, float* state, long long state_stride, const int* cu_q,
                                   const int* req_slots, const int* token_req, float* out, int tokens, int requests,
                                   int heads, int dim, int vdim, int num_slots, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (requests < 0 || tokens < 0 || heads <= 0 || dim <= 0 || vdim <= 0 || num_slots <= 0) return ULLM_ERR_BAD_SIZE;
  if (dim > GLA_MAX_DIM || heads > 65535 || requests > 65535) return ULLM_ERR_UNSUPPORTED;
  if (state_stride < (long long)heads * vdim * dim) return ULLM_ERR_BAD_SIZE;
  if (requests == 0) return ULLM_OK;
#define GLA_ARGS                                                                                                     \
  qkv, row_stride, q_off, k_off, v_off, z, z_stride, z_bias, inv_tau, q_scale, state, state_stride, cu_q, req_slots, \
      token_req, out, tokens, requests, heads, dim, vdim, num_slots, status, st
  if (dtype == ULLM_DTYPE_F32) return gla_launch<float>(GLA_ARGS);
  if (dtype == ULLM_DTYPE_BF16) return gla_launch<__nv_bfloat16>(GLA_ARGS);
  if (dtype == ULLM_DTYPE_F16) return gla_launch<__half>(GLA_ARGS);
#undef GLA_ARGS
  return ULLM_ERR_BAD_DTYPE;
}
