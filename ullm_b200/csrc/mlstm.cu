// Matrix memory with exponential gates (the mLSTM recurrence), for any mix of
// requests in one flat batch: prompt portions of any length beside single
// decoded tokens.  Per request and head the state is a matrix S [d, dv], a
// vector n [d] and a running maximum m, all 32-bit, kept in the request's state
// row between steps:
//
//   i_t = cap tanh((a_t + b_i) / cap)                     log input gate (a, c: the gate projections)
//   f_t = logsigmoid(cap tanh((c_t + b_f) / cap))         log forget gate
//   m_t = max(f_t + m_{t-1}, i_t)
//   S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T      (n_t alike with k_t alone)
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),   q_t = q_scale * (projected query)
//
// The recurrence is run token by token, so a request's result does not depend on how its tokens were cut into
// steps.  The parallelism is over requests, heads and the columns of S: a block owns (request, head, a tile of
// columns); a column's d rows are spread over RS neighbouring lanes (row r belongs to lane r mod RS), which meet
// in shuffles for the two dot products.  q, k and the tile's v of a chunk of tokens are staged in shared memory,
// and the chunk's gates, running maximum and the three exponentials of every token evaluated, by a second set of
// threads of the block while the first set runs the chunk before (two buffers): the first set is left with the
// multiply-adds, the shuffles and one division per token.
//
// State row layout (floats): S^T as [heads][dv][d], then n [heads][d], then m [heads].
//
// A second kernel finishes the mixer's head: per (token, head) o / sqrt(mean(o^2) + eps) * w * sigmoid(g).
#include "common.cuh"

#include <type_traits>

#define MLSTM_THREADS 128
#define MLSTM_RPT 16       // rows of S a thread holds at most
#define MLSTM_MAX_DIM 512  // = 32 lanes * MLSTM_RPT

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// RPT: rows of S a thread holds at most (8 or MLSTM_RPT).  RS > 0: the lanes per column are known when the kernel
// is compiled and dim == RS * RPT exactly, so the row loop has neither bounds checks nor address arithmetic left
// (measured at dim 128: 2.5 times fewer instructions per token); RS == 0: any dim, lanes per column in `rs_arg`.
// CPT: neighbouring value columns a thread holds (1 or 4): the k and q a thread reads from shared memory and its
// share of n serve all of them, which is what the multiply-adds wait for otherwise.
template <typename T, int RPT, int RS, int CPT>
__global__ void __launch_bounds__(2 * MLSTM_THREADS)
mlstm_recurrence_kernel(const T* __restrict__ qkv, long long row_stride, int q_off, int k_off, int v_off,
                        const float* __restrict__ gates, const float* __restrict__ bias_i,
                        const float* __restrict__ bias_f, float* __restrict__ state, long long state_stride,
                        const int* __restrict__ cu_q, const int* __restrict__ req_slots,
                        const int* __restrict__ token_req, float* __restrict__ out, int heads, int dim, int vdim,
                        int rs_arg, int chunk, float q_scale, float cap, int num_slots, int* status) {
  constexpr bool FULL = RS != 0;
  const int rs = FULL ? RS : rs_arg;
  // Threads 0 .. 127 run the recurrence; threads 128 .. 255 stage the next chunk of tokens (q, k, the tile's v,
  // the evaluated gates) in the other half of shared memory meanwhile, so the recurrence never waits for memory.
  extern __shared__ float sm[];
  pdl_launch_dependents();
  pdl_wait();
  const int req = blockIdx.z, head = blockIdx.y;
  const int cols_per_block = (MLSTM_THREADS / rs) * CPT;
  const bool loader = threadIdx.x >= MLSTM_THREADS;
  const int tid = threadIdx.x & (MLSTM_THREADS - 1);
  const int lane_row = tid % rs;          // which rows: lane_row, lane_row + rs, ...
  const int col_in_block = tid / rs;
  const int col = blockIdx.x * cols_per_block + col_in_block * CPT;  // the thread's first column
  const bool col_ok = col < vdim;
  const int t0 = cu_q[req], t1 = cu_q[req + 1];
  if (t1 <= t0) return;
  const bool padding = token_req[t0] < 0;  // a row that belongs to no request: zeros out, no state touched
  const int slot = req_slots[req];
  if (!padding && (slot < 0 || slot >= num_slots)) {
    if (threadIdx.x == 0) ullm_report(status, ULLM_STATUS_SLOT, req, slot);
    return;
  }
  if (padding) {
    if (!loader && lane_row == 0)
      for (int t = t0; t < t1; ++t)
        for (int c = 0; c < CPT; ++c)
          if (col + c < vdim) out[((long long)t * heads + head) * vdim + col + c] = 0.f;
    return;
  }
  const int buf_floats = (2 * chunk * dim + chunk * cols_per_block + 3 * chunk + 1 + 3) & ~3;  // (16-byte steps)
  const bool vec8 = std::is_same<T, __nv_bfloat16>::value && (dim & 7) == 0 && (q_off & 7) == 0 && (k_off & 7) == 0 && (row_stride & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(qkv) & 15) == 0;
  const float bi = bias_i != nullptr ? bias_i[head] : 0.f, bf = bias_f != nullptr ? bias_f[head] : 0.f;

  float* st_row = state + (long long)slot * state_stride;
  float* st_S = st_row + ((long long)head * vdim + (col_ok ? col : 0)) * dim;  // column c of the thread: + c * dim
  float* st_n = st_row + (long long)heads * vdim * dim + (long long)head * dim;
  float* st_m = st_row + (long long)heads * vdim * dim + (long long)heads * dim + head;

  float m_run = *st_m;  // the running maximum as the stagers carry it, one chunk ahead of the recurrence

  // stages tokens c0 .. c0 + cn - 1 into buffer `which` (loader threads only)
  auto fill = [&](int which, int c0, int cn) {
    float* sq = sm + which * buf_floats;   // [chunk][dim]
    float* sk = sq + chunk * dim;          // [chunk][dim]
    float* sv = sk + chunk * dim;          // [chunk][cols_per_block]
    float* s_keep = sv + chunk * cols_per_block;  // exp(f_t + m_{t-1} - m_t)
    float* s_take = s_keep + chunk;               // exp(i_t - m_t)
    float* s_einv = s_take + chunk;               // exp(-m_t); then one float: m after the chunk
    const int n_qk = cn * dim;
    if (vec8) {
      // bfloat16 rows that allow 16-byte pieces: a thread moves 8 neighbouring elements of q and of k per load
      const int per_tok = dim >> 3, n8 = cn * per_tok;
      for (int g0 = tid; g0 < n8; g0 += MLSTM_THREADS * 4) {
        uint4 rq[4], rk[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int g = g0 + j * MLSTM_THREADS;
          if (g < n8) {
            const int t = g / per_tok, r = (g - t * per_tok) << 3;
            const T* row = qkv + (long long)(c0 + t) * row_stride + head * dim + r;
            rq[j] = *reinterpret_cast<const uint4*>(row + q_off);
            rk[j] = *reinterpret_cast<const uint4*>(row + k_off);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int g = g0 + j * MLSTM_THREADS;
          if (g < n8) {
            const __nv_bfloat16* eq = reinterpret_cast<const __nv_bfloat16*>(&rq[j]);
            const __nv_bfloat16* ek = reinterpret_cast<const __nv_bfloat16*>(&rk[j]);
            float4 a, b, c, d;
            a.x = __bfloat162float(eq[0]) * q_scale, a.y = __bfloat162float(eq[1]) * q_scale;
            a.z = __bfloat162float(eq[2]) * q_scale, a.w = __bfloat162float(eq[3]) * q_scale;
            b.x = __bfloat162float(eq[4]) * q_scale, b.y = __bfloat162float(eq[5]) * q_scale;
            b.z = __bfloat162float(eq[6]) * q_scale, b.w = __bfloat162float(eq[7]) * q_scale;
            c.x = __bfloat162float(ek[0]), c.y = __bfloat162float(ek[1]), c.z = __bfloat162float(ek[2]), c.w = __bfloat162float(ek[3]);
            d.x = __bfloat162float(ek[4]), d.y = __bfloat162float(ek[5]), d.z = __bfloat162float(ek[6]), d.w = __bfloat162float(ek[7]);
            const int t = g / per_tok, e = t * dim + ((g - t * per_tok) << 3);
            *reinterpret_cast<float4*>(sq + e) = a;
            *reinterpret_cast<float4*>(sq + e + 4) = b;
            *reinterpret_cast<float4*>(sk + e) = c;
            *reinterpret_cast<float4*>(sk + e + 4) = d;
          }
        }
      }
    } else
    for (int e0 = tid; e0 < n_qk; e0 += MLSTM_THREADS * 8) {
      float tq[8], tk[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = e0 + j * MLSTM_THREADS;
        if (e < n_qk) {
          const int t = e / dim, r = e - t * dim;
          const T* row = qkv + (long long)(c0 + t) * row_stride + head * dim + r;
          tq[j] = to_f32(row[q_off]);
          tk[j] = to_f32(row[k_off]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = e0 + j * MLSTM_THREADS;
        if (e < n_qk) {
          sq[e] = tq[j] * q_scale;
          sk[e] = tk[j];
        }
      }
    }
    const int n_v = cn * cols_per_block;
    for (int e0 = tid; e0 < n_v; e0 += MLSTM_THREADS * 4) {
      float tv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + j * MLSTM_THREADS;
        tv[j] = 0.f;
        if (e < n_v) {
          const int t = e / cols_per_block, cj = blockIdx.x * cols_per_block + (e - t * cols_per_block);
          if (cj < vdim) tv[j] = to_f32(qkv[(long long)(c0 + t) * row_stride + v_off + head * vdim + cj]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + j * MLSTM_THREADS;
        if (e < n_v) sv[e] = tv[j];
      }
    }
    // The gates and the running maximum of the chunk: a scan of a few tokens, by one warp of the stagers (the
    // lanes evaluate the gates side by side, lane 0 runs the maximum along), so that the recurrence itself is
    // left with multiply-adds.  `m_run` carries the maximum from chunk to chunk (it starts at the state's).
    if (tid < 32) {
      float gi = 0.f, gf = 0.f;
      if (tid < cn) {
        const float* g = gates + (long long)(c0 + tid) * 2 * heads;
        gi = cap * tanhf((g[head] + bi) / cap);
        gf = log_sigmoid(cap * tanhf((g[heads + head] + bf) / cap));
      }
      for (int t = 0; t < cn; ++t) {
        const float ii = __shfl_sync(0xffffffffu, gi, t), fi = __shfl_sync(0xffffffffu, gf, t);
        const float m_new = fmaxf(fi + m_run, ii);
        if (tid == 0) {
          s_keep[t] = expf(fi + m_run - m_new);
          s_take[t] = expf(ii - m_new);
          s_einv[t] = expf(-m_new);
        }
        m_run = m_new;
      }
      if (tid == 0) s_einv[chunk] = m_run;
    }
  };

  float S[RPT][CPT], n[RPT];
  float m = 0.f;
  if (!loader) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int r = lane_row + rs * i;
      const bool on = r < dim;
#pragma unroll
      for (int c = 0; c < CPT; ++c) S[i][c] = (on && col + c < vdim) ? st_S[(long long)c * dim + r] : 0.f;
      n[i] = on ? st_n[r] : 0.f;
    }
    m = *st_m;
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
      const float* sk = sq + chunk * dim;
      const float* sv = sk + chunk * dim;
      const float* s_keep = sv + chunk * cols_per_block;
      const float* s_take = s_keep + chunk;
      const float* s_einv = s_take + chunk;
#pragma unroll 2
      for (int t = 0; t < cn; ++t) {
        const float keep = s_keep[t], take = s_take[t];
        float tv[CPT];
#pragma unroll
        for (int c = 0; c < CPT; ++c) tv[c] = take * sv[t * cols_per_block + col_in_block * CPT + c];
        const float* kq = sk + t * dim;
        const float* qq = sq + t * dim;
        float dot[2][CPT], ndot[2] = {0.f, 0.f};  // rows of even and of odd index into sums of their own
#pragma unroll
        for (int c = 0; c < CPT; ++c) dot[0][c] = dot[1][c] = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int r = lane_row + rs * i;
          if (FULL || r < dim) {
            const float kr = kq[r], qr = qq[r];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
              S[i][c] = fmaf(keep, S[i][c], kr * tv[c]);
              dot[i & 1][c] = fmaf(S[i][c], qr, dot[i & 1][c]);
            }
            n[i] = fmaf(keep, n[i], take * kr);
            ndot[i & 1] = fmaf(n[i], qr, ndot[i & 1]);
          }
        }
        float nd = ndot[0] + ndot[1];
#pragma unroll
        for (int c = 0; c < CPT; ++c) dot[0][c] += dot[1][c];
        if (FULL) {
#pragma unroll
          for (int o = RS >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int c = 0; c < CPT; ++c) dot[0][c] += __shfl_xor_sync(0xffffffffu, dot[0][c], o);
            nd += __shfl_xor_sync(0xffffffffu, nd, o);
          }
        } else {
          for (int o = rs >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int c = 0; c < CPT; ++c) dot[0][c] += __shfl_xor_sync(0xffffffffu, dot[0][c], o);
            nd += __shfl_xor_sync(0xffffffffu, nd, o);
          }
        }
        if (lane_row == 0) {
          const float den = fmaxf(fabsf(nd), s_einv[t]) + 1e-6f;
#pragma unroll
          for (int c = 0; c < CPT; ++c)
            if (col + c < vdim) out[((long long)(c0 + t) * heads + head) * vdim + col + c] = dot[0][c] / den;
        }
      }
      m = s_einv[chunk];
    }
    __syncthreads();  // the next chunk is staged, this one used up
  }
  if (loader) return;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = lane_row + rs * i;
    if (r < dim) {
#pragma unroll
      for (int c = 0; c < CPT; ++c)
        if (col + c < vdim) st_S[(long long)c * dim + r] = S[i][c];
      if (blockIdx.x == 0 && col_in_block == 0) st_n[r] = n[i];
    }
  }
  if (blockIdx.x == 0 && tid == 0) *st_m = m;
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w[h, :] * sigmoid(g[t, h, :]); one warp per (token, head).
template <typename T>
__global__ void mlstm_out_gate_kernel(const float* __restrict__ o, const T* __restrict__ g, long long g_stride,
                                      const float* __restrict__ w, T* __restrict__ out, long long units, int heads,
                                      int vdim, float eps, int w_per_head, int silu) {
  pdl_launch_dependents();
  pdl_wait();
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= units) return;
  const long long t = unit / heads;
  const int h = (int)(unit - t * heads);
  const float* src = o + unit * vdim;
  float ss = 0.f;
  for (int e = lane; e < vdim; e += 32) ss += src[e] * src[e];
  ss = warp_sum(ss);
  const float rstd = 1.f / sqrtf(ss / (float)vdim + eps);
  const T* gr = g + t * g_stride + (long long)h * vdim;
  for (int e = lane; e < vdim; e += 32) {
    const float gv = to_f32(gr[e]);
    const float gate = (silu ? gv : 1.f) / (1.f + expf(-gv));
    out[unit * vdim + e] = from_f32<T>(src[e] * rstd * w[(w_per_head ? h * vdim : 0) + e] * gate);
  }
}

// Lanes that share a column: as many as leave a thread about 8 rows (the per-token chain of a thread is what
// paces the recurrence, and narrower column tiles make more blocks), at most a warp.
static int mlstm_rs(int dim) {
  int rs = 1;
  while (rs < 32 && rs * 8 < dim) rs <<= 1;
  return rs;
}

extern "C" int ullm_mlstm_supported(int heads, int dim, int vdim) {
  return heads > 0 && dim > 0 && vdim > 0 && dim <= MLSTM_MAX_DIM;
}

// Floats of one request's state row.
extern "C" long long ullm_mlstm_state_floats(int heads, int dim, int vdim) {
  return (long long)heads * vdim * dim + (long long)heads * dim + heads;
}

template <typename T>
static int mlstm_launch(const void* qkv, long long row_stride, int q_off, int k_off, int v_off, const float* gates,
                        const float* bias_i, const float* bias_f, float* state, long long state_stride,
                        const int* cu_q, const int* req_slots, const int* token_req, float* out, int requests,
                        int heads, int dim, int vdim, float q_scale, float cap, int num_slots, int* status,
                        cudaStream_t st) {
  const int rs = mlstm_rs(dim);
  // four (or two) columns per thread where that still leaves the SMs about two blocks each (fewer, fatter blocks: less
  // q / k staging, several multiply-add chains per row read: head size 256 x 512, one prompt of 2,048 tokens,
  // 13.6 -> 5.7 ms for four layers; but 256 values wide at one request, 64 blocks of four columns were slower
  // than 256 of one)
  int cpt = 1;
  for (int c = 4; c > 1; c >>= 1) {
    const int tile = (MLSTM_THREADS / rs) * c;
    if (vdim >= tile && (long long)((vdim + tile - 1) / tile) * heads * requests >= 250) {
      cpt = c;
      break;
    }
  }
  const int cols = (MLSTM_THREADS / rs) * cpt;
  // tokens per staged chunk: two buffers of (2 dim + cols + 2) floats a token stay below 48 KB
  int chunk = 16;
  while (chunk > 1 && (size_t)2 * chunk * (2 * dim + cols + 3) * sizeof(float) > 46 * 1024) chunk >>= 1;
  const size_t smem = (size_t)2 * ((2 * chunk * dim + chunk * cols + 3 * chunk + 1 + 3) & ~3) * sizeof(float);
  const dim3 grid((vdim + cols - 1) / cols, heads, requests);
#define MLSTM_LAUNCH(RPT_, RS_)                                                                                       \
  do {                                                                                                                \
    if (cpt == 4)                                                                                                     \
      return ullm_launch_kernel(mlstm_recurrence_kernel<T, RPT_, RS_, 4>, grid, dim3(2 * MLSTM_THREADS), smem, st,     \
                                (const T*)qkv, row_stride, q_off, k_off, v_off, gates, bias_i, bias_f, state,         \
                                state_stride, cu_q, req_slots, token_req, out, heads, dim, vdim, rs, chunk, q_scale,   \
                                cap, num_slots, status);                                                              \
    if (cpt == 2)                                                                                                     \
      return ullm_launch_kernel(mlstm_recurrence_kernel<T, RPT_, RS_, 2>, grid, dim3(2 * MLSTM_THREADS), smem, st,     \
                                (const T*)qkv, row_stride, q_off, k_off, v_off, gates, bias_i, bias_f, state,         \
                                state_stride, cu_q, req_slots, token_req, out, heads, dim, vdim, rs, chunk, q_scale,   \
                                cap, num_slots, status);                                                              \
    return ullm_launch_kernel(mlstm_recurrence_kernel<T, RPT_, RS_, 1>, grid, dim3(2 * MLSTM_THREADS), smem, st,       \
                              (const T*)qkv, row_stride, q_off, k_off, v_off, gates, bias_i, bias_f, state,           \
                              state_stride, cu_q, req_slots, token_req, out, heads, dim, vdim, rs, chunk, q_scale,     \
                              cap, num_slots, status);                                                                \
  } while (0)
  if (dim == 64 && rs == 8) MLSTM_LAUNCH(8, 8);
  if (dim == 128 && rs == 16) MLSTM_LAUNCH(8, 16);
  if (dim == 256 && rs == 32) MLSTM_LAUNCH(8, 32);
  if (dim == 512 && rs == 32) MLSTM_LAUNCH(16, 32);
  if (rs * 8 >= dim) MLSTM_LAUNCH(8, 0);
  MLSTM_LAUNCH(MLSTM_RPT, 0);
#undef MLSTM_LAUNCH
}

// qkv: rows of `row_stride` elements that hold q [heads, dim] at q_off, k [heads, dim] at k_off and v [heads, vdim]
// at v_off.  gates: [tokens, 2 heads] float32, the input-gate projections then the forget-gate projections (biases
// not yet added).  state: [num_slots, state_stride] float32.  out: [tokens, heads, vdim] float32.
extern "C" int ullm_mlstm_recurrence(int dtype, const void* qkv, long long row_stride, int q_off, int k_off,
                                     int v_off, const float* gates, const float* bias_i, const float* bias_f,
                                     float* state, long long state_stride, const int* cu_q, const int* req_slots,
                                     const int* token_req, float* out, int requests, int heads, int dim, int vdim,
                                     float q_scale, float cap, int num_slots, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (requests < 0 || !ullm_mlstm_supported(heads, dim, vdim)) return ULLM_ERR_UNSUPPORTED;
  if (state_stride < ullm_mlstm_state_floats(heads, dim, vdim) || cap <= 0.f) return ULLM_ERR_BAD_SIZE;
  if (requests == 0) return ULLM_OK;
  if (requests > 65535 || heads > 65535) return ULLM_ERR_BAD_SIZE;
  if (dtype == ULLM_DTYPE_F32)
    return mlstm_launch<float>(qkv, row_stride, q_off, k_off, v_off, gates, bias_i, bias_f, state, state_stride,
                               cu_q, req_slots, token_req, out, requests, heads, dim, vdim, q_scale, cap, num_slots,
                               status, st);
  if (dtype == ULLM_DTYPE_BF16)
    return mlstm_launch<__nv_bfloat16>(qkv, row_stride, q_off, k_off, v_off, gates, bias_i, bias_f, state,
                                       state_stride, cu_q, req_slots, token_req, out, requests, heads, dim, vdim,
                                       q_scale, cap, num_slots, status, st);
  if (dtype == ULLM_DTYPE_F16)
    return mlstm_launch<__half>(qkv, row_stride, q_off, k_off, v_off, gates, bias_i, bias_f, state, state_stride,
                                cu_q, req_slots, token_req, out, requests, heads, dim, vdim, q_scale, cap, num_slots,
                                status, st);
  return ULLM_ERR_BAD_DTYPE;
}

// Per (token, head): o / sqrt(mean(o^2) + eps) * w * gate(g), with w [heads * vdim] (`w_per_head`) or [vdim] shared
// by the heads, and gate = sigmoid (`silu` 0) or silu (1).
extern "C" int ullm_head_norm_gate(int dtype, const float* o, const void* g, long long g_stride, const float* w,
                                   void* out, int tokens, int heads, int vdim, float eps, int w_per_head, int silu,
                                   void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || heads <= 0 || vdim <= 0) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  const long long units = (long long)tokens * heads;
  const long long blocks = (units + 3) / 4;
  if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
  const dim3 grid((int)blocks), block(128);
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(mlstm_out_gate_kernel<float>, grid, block, 0, st, o, (const float*)g, g_stride, w,
                              (float*)out, units, heads, vdim, eps, w_per_head, silu);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(mlstm_out_gate_kernel<__nv_bfloat16>, grid, block, 0, st, o, (const __nv_bfloat16*)g,
                              g_stride, w, (__nv_bfloat16*)out, units, heads, vdim, eps, w_per_head, silu);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(mlstm_out_gate_kernel<__half>, grid, block, 0, st, o, (const __half*)g, g_stride, w,
                              (__half*)out, units, heads, vdim, eps, w_per_head, silu);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_mlstm_out_gate(int dtype, const float* o, const void* g, long long g_stride, const float* w,
                                   void* out, int tokens, int heads, int vdim, float eps, void* stream) {
  return ullm_head_norm_gate(dtype, o, g, g_stride, w, out, tokens, heads, vdim, eps, 1, 0, stream);
}
