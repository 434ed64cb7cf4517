// What lies between an attention's q | k | v projection and its scores, in its general form, for any mix of
// requests in one flat batch (prompt portions beside single decoded tokens):
//
//   1. optionally a short causal convolution over time on every channel of q, k and v:
//        y_t[c] = sum_j w[c][j] u_(t - taps + 1 + j)[c]
//      The taps - 1 projected rows that precede a step's first token come from the request's state row
//      ([taps - 1][row width] floats, zeros for a new request; row s holds the token taps - 1 - s places before
//      the step's first).  `conv_state_update` moves the state on after the step.
//   2. optionally a per-head RMS norm of q and k BEFORE the rotation, with or without a weight;
//   3. the rotation of the first `rotary_dim` dimensions of every q and k head, dimension i with dimension
//      i + rotary_dim / 2, by the angle position * inv_freq[i] (the 32-bit product; sincosf with full range
//      reduction: no table per position, no largest position);
//   4. optionally the unit RMS norm of q and k AFTER the rotation (no weight);
//   5. optionally value mixing across layers: the first layer that mixes leaves its values of the step's tokens
//      in `v_first`, every later one computes v <- (1 - lambda) v + lambda v_first;
//   6. k and v go to their cache slots, q to `q_out` [T, heads * head_dim].
//
// One warp per (token, head) over the q heads, the k heads and the v heads.  All arithmetic is 32-bit; a value is
// rounded once, when it is stored.
#include "common.cuh"

#define PREP_MAX_DIM 512
#define PREP_WARPS 4
#define PREP_MAX_TAPS 32

template <typename T>
__global__ void qkv_prepare_kernel(const T* __restrict__ qkv, long long row_stride, int tokens, int num_q, int num_kv,
                                   int head_dim, int v_dim, const T* __restrict__ conv_w, int taps,
                                   const float* __restrict__ conv_state, long long state_stride,
                                   const int* __restrict__ cu_q, const int* __restrict__ token_req,
                                   const int* __restrict__ req_slots, int num_state_slots,
                                   const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                   int rotary_dim, const float* __restrict__ q_w, const float* __restrict__ k_w,
                                   int norm_first, int norm_last, float eps, int vmix_mode,
                                   const float* __restrict__ vmix_lambda, T* __restrict__ v_first,
                                   const int* __restrict__ slot_mapping, T* __restrict__ k_cache,
                                   T* __restrict__ v_cache, long long num_slots, T* __restrict__ q_out, int* status) {
  __shared__ float buf[PREP_WARPS][PREP_MAX_DIM];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units_per_token = num_q + 2 * num_kv;
  const long long unit = (long long)blockIdx.x * PREP_WARPS + warp;
  if (unit >= (long long)tokens * units_per_token) return;
  const int t = (int)(unit / units_per_token);
  const int u = (int)(unit - (long long)t * units_per_token);
  const int kind = u < num_q ? 0 : (u < num_q + num_kv ? 1 : 2);  // q, k, v
  const int head = kind == 0 ? u : (kind == 1 ? u - num_q : u - num_q - num_kv);
  const int dim = kind == 2 ? v_dim : head_dim;
  const int q_size = num_q * head_dim, k_size = num_kv * head_dim;
  const int chan0 = (kind == 0 ? 0 : (kind == 1 ? q_size : q_size + k_size)) + head * dim;  // column in the row
  const int r = token_req[t];
  float* x = buf[warp];

  // 1. the projected values, through the short convolution if there is one
  if (conv_w != nullptr && r >= 0) {
    const int t0 = cu_q[r];
    const int slot = req_slots[r];
    const bool slot_ok = taps > 1 && slot >= 0 && slot < num_state_slots;  // (one tap: no memory, no state row)
    if (taps > 1 && !slot_ok && lane == 0) ullm_report(status, ULLM_STATUS_SLOT, t, slot);
    const float* st = conv_state + (long long)(slot_ok ? slot : 0) * state_stride;
    const int row_width = q_size + k_size + num_kv * v_dim;
    for (int e = lane; e < dim; e += 32) {
      const int c = chan0 + e;
      float y = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;  // tokens before this one
        const int row = t - back;
        float uval;
        if (row >= t0) {
          uval = to_f32(qkv[(long long)row * row_stride + c]);
        } else {
          const int s = taps - 1 - (t0 - row);  // t0 - row in 1 .. taps - 1
          uval = slot_ok ? st[(long long)s * row_width + c] : 0.f;
        }
        y += to_f32(conv_w[(long long)c * taps + j]) * uval;
      }
      x[e] = y;
    }
  } else {
    for (int e = lane; e < dim; e += 32) x[e] = to_f32(qkv[(long long)t * row_stride + chan0 + e]);
  }
  __syncwarp();

  if (kind == 2) {
    // 5. value mixing, then the cache
    T* vf = v_first != nullptr ? v_first + (long long)t * num_kv * v_dim + head * v_dim : nullptr;
    const float lam = vmix_mode == 2 ? *vmix_lambda : 0.f;
    const int slot = slot_mapping != nullptr ? slot_mapping[t] : -1;
    const bool store = slot >= 0 && slot < num_slots;
    if (slot_mapping != nullptr && slot >= num_slots && lane == 0) ullm_report(status, ULLM_STATUS_SLOT, t, slot);
    T* dst = store ? v_cache + ((long long)slot * num_kv + head) * v_dim : nullptr;
    for (int e = lane; e < dim; e += 32) {
      float v = x[e];
      if (vmix_mode == 2) v = (1.f - lam) * v + lam * to_f32(vf[e]);
      const T rounded = from_f32<T>(v);
      if (vmix_mode == 1) vf[e] = rounded;
      if (store) dst[e] = rounded;
    }
    return;
  }

  const float* w = kind == 0 ? q_w : k_w;
  // 2. norm in front of the rotation
  if (norm_first) {
    float ss = 0.f;
    for (int e = lane; e < dim; e += 32) ss += x[e] * x[e];
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)dim + eps);
    for (int e = lane; e < dim; e += 32) x[e] = x[e] * rstd * (w != nullptr ? w[e] : 1.f);
    __syncwarp();
  }
  // 3. rotation
  if (rotary_dim > 0 && inv_freq != nullptr) {
    const float p = (float)positions[t];
    const int half = rotary_dim >> 1;
    for (int i = lane; i < half; i += 32) {
      float sn, cs;
      sincosf(p * inv_freq[i], &sn, &cs);
      const float a = x[i], b = x[i + half];
      x[i] = a * cs - b * sn;
      x[i + half] = b * cs + a * sn;
    }
    __syncwarp();
  }
  // 4. unit norm behind the rotation
  float mult = 1.f;
  if (norm_last) {
    float ss = 0.f;
    for (int e = lane; e < dim; e += 32) ss += x[e] * x[e];
    ss = warp_sum(ss);
    mult = 1.f / sqrtf(ss / (float)dim + eps);
  }
  // 6. stores
  if (kind == 0) {
    T* dst = q_out + ((long long)t * num_q + head) * head_dim;
    for (int e = lane; e < dim; e += 32) dst[e] = from_f32<T>(x[e] * mult);
  } else {
    const int slot = slot_mapping != nullptr ? slot_mapping[t] : -1;
    if (slot_mapping != nullptr && slot >= num_slots && lane == 0) ullm_report(status, ULLM_STATUS_SLOT, t, slot);
    if (slot >= 0 && slot < num_slots) {
      T* dst = k_cache + ((long long)slot * num_kv + head) * head_dim;
      for (int e = lane; e < dim; e += 32) dst[e] = from_f32<T>(x[e] * mult);
    }
  }
}

// After a step: the state row of every request of the step holds the last taps - 1 projected rows.  One thread
// per (request, channel); rows are moved in ascending order, so a request that brought fewer than taps - 1 tokens
// shifts its old rows down before it appends (row s takes old row s + n: always a row not yet written).
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ qkv, long long row_stride, int row_width, int taps,
                                         float* __restrict__ conv_state, long long state_stride,
                                         const int* __restrict__ cu_q, const int* __restrict__ token_req,
                                         const int* __restrict__ req_slots, int num_state_slots, int requests) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  if (r >= requests) return;
  const int t0 = cu_q[r], t1 = cu_q[r + 1];
  const int n = t1 - t0;
  if (n <= 0 || token_req[t0] < 0) return;  // a padding row belongs to no request
  const int slot = req_slots[r];
  if (slot < 0 || slot >= num_state_slots) return;
  float* st = conv_state + (long long)slot * state_stride;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < row_width; c += gridDim.x * blockDim.x) {
    for (int s = 0; s < taps - 1; ++s) {
      const int back = taps - 1 - s;  // rows before the end
      float v;
      if (back <= n) v = to_f32(qkv[(long long)(t1 - back) * row_stride + c]);
      else v = st[(long long)(s + n) * row_width + c];
      st[(long long)s * row_width + c] = v;
    }
  }
}

template <typename T>
static int prepare_launch(const void* qkv, long long row_stride, int tokens, int num_q, int num_kv, int head_dim,
                          int v_dim, const void* conv_w, int taps, const float* conv_state, long long state_stride,
                          const int* cu_q, const int* token_req, const int* req_slots, int num_state_slots,
                          const int* positions, const float* inv_freq, int rotary_dim, const float* q_w,
                          const float* k_w, int norm_first, int norm_last, float eps, int vmix_mode,
                          const float* vmix_lambda, void* v_first, const int* slot_mapping, void* k_cache,
                          void* v_cache, long long num_slots, void* q_out, int* status, cudaStream_t st) {
  const long long units = (long long)tokens * (num_q + 2 * num_kv);
  const long long blocks = (units + PREP_WARPS - 1) / PREP_WARPS;
  if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
  return ullm_launch_kernel(qkv_prepare_kernel<T>, dim3((int)blocks), dim3(PREP_WARPS * 32), 0, st, (const T*)qkv,
                            row_stride, tokens, num_q, num_kv, head_dim, v_dim, (const T*)conv_w, taps, conv_state,
                            state_stride, cu_q, token_req, req_slots, num_state_slots, positions, inv_freq, rotary_dim,
                            q_w, k_w, norm_first, norm_last, eps, vmix_mode, vmix_lambda, (T*)v_first, slot_mapping,
                            (T*)k_cache, (T*)v_cache, num_slots, (T*)q_out, status);
}

// `conv_w`: [row width][taps] in the engine's dtype (the q, k and v filters one after the other) or null.
// `vmix_mode`: 0 none, 1 this layer leaves its values in `v_first`, 2 it mixes them in with *vmix_lambda.
extern "C" int ullm_qkv_prepare(int dtype, const void* qkv, long long row_stride, int tokens, int num_q, int num_kv,
                                int head_dim, int v_dim, const void* conv_w, int taps, const float* conv_state,
                                long long state_stride, const int* cu_q, const int* token_req, const int* req_slots,
                                int num_state_slots, const int* positions, const float* inv_freq, int rotary_dim,
                                const float* q_w, const float* k_w, int norm_first, int norm_last, float eps,
                                int vmix_mode, const float* vmix_lambda, void* v_first, const int* slot_mapping,
                                void* k_cache, void* v_cache, long long num_slots, void* q_out, int* status,
                                void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0 || v_dim <= 0) return ULLM_ERR_BAD_SIZE;
  if (head_dim > PREP_MAX_DIM || v_dim > PREP_MAX_DIM || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
    return ULLM_ERR_UNSUPPORTED;
  if (conv_w != nullptr && (taps < 1 || taps > PREP_MAX_TAPS || (taps > 1 && conv_state == nullptr)))
    return ULLM_ERR_UNSUPPORTED;
  if (vmix_mode < 0 || vmix_mode > 2 || (vmix_mode != 0 && v_first == nullptr) ||
      (vmix_mode == 2 && vmix_lambda == nullptr))
    return ULLM_ERR_BAD_SIZE;
  if (rotary_dim > 0 && (inv_freq == nullptr || positions == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
#define PREP_ARGS                                                                                                   \
  qkv, row_stride, tokens, num_q, num_kv, head_dim, v_dim, conv_w, taps, conv_state, state_stride, cu_q, token_req,  \
      req_slots, num_state_slots, positions, inv_freq, rotary_dim, q_w, k_w, norm_first, norm_last, eps, vmix_mode, \
      vmix_lambda, v_first, slot_mapping, k_cache, v_cache, num_slots, q_out, status, st
  if (dtype == ULLM_DTYPE_F32) return prepare_launch<float>(PREP_ARGS);
  if (dtype == ULLM_DTYPE_BF16) return prepare_launch<__nv_bfloat16>(PREP_ARGS);
  if (dtype == ULLM_DTYPE_F16) return prepare_launch<__half>(PREP_ARGS);
#undef PREP_ARGS
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_conv_state_update(int dtype, const void* qkv, long long row_stride, int row_width, int taps,
                                      float* conv_state, long long state_stride, const int* cu_q,
                                      const int* token_req, const int* req_slots, int num_state_slots, int requests,
                                      void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (requests < 0 || row_width <= 0 || taps < 1 || taps > PREP_MAX_TAPS) return ULLM_ERR_BAD_SIZE;
  if (requests == 0 || taps == 1) return ULLM_OK;
  if (requests > 65535) return ULLM_ERR_UNSUPPORTED;
  const dim3 grid((row_width + 127) / 128, requests), block(128);
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(conv_state_update_kernel<float>, grid, block, 0, st, (const float*)qkv, row_stride,
                              row_width, taps, conv_state, state_stride, cu_q, token_req, req_slots, num_state_slots,
                              requests);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(conv_state_update_kernel<__nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)qkv,
                              row_stride, row_width, taps, conv_state, state_stride, cu_q, token_req, req_slots,
                              num_state_slots, requests);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(conv_state_update_kernel<__half>, grid, block, 0, st, (const __half*)qkv, row_stride,
                              row_width, taps, conv_state, state_stride, cu_q, token_req, req_slots, num_state_slots,
                              requests);
  return ULLM_ERR_BAD_DTYPE;
}
