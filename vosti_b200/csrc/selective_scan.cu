// Selective scan (the Mamba mixer's recurrence) with its short convolution.
//
// Per request a state slot holds S [inner, N] (float32) and the convolution's last taps - 1
// inputs [taps - 1, inner] (float32). For every token, channel c and state n:
//
//   x_c   = silu(conv(u)_c)                        u: the first half of the input projection
//   dt_c  = softplus(dtp_c + dt_bias_c)            dtp: the step-size projection (float32)
//   S[c,n] <- exp(dt_c * A[c,n]) * S[c,n] + dt_c * x_c * B_n,   A = -exp(A_log)
//   y_c   = (sum_n S[c,n] * C_n + D_c * x_c) * silu(z_c)       z: the second half of the input projection
//
// Kernels:
//   scan_conv   convolution + SiLU for every token of the step (block per token); a token near the start
//               of its request's portion takes the inputs before the portion from the slot's tail.
//   scan_tail   the tail after this step, one thread per (request, channel); it runs after
//               scan_conv has read the old tail.
//   scan_run    the recurrence: a block per (request, 32 channels), LANES lanes share a channel and
//               split its states; tokens in order, the next token's inputs loaded while this one's
//               are used. Everything after the projections is float32.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename T>
__global__ void __launch_bounds__(256)
scan_conv_kernel(const T* __restrict__ xz, int64_t xz_stride, const void* __restrict__ conv_w, const void* __restrict__ conv_b,
                 int w_f32, const float* state, int64_t state_stride, int64_t tail_offset, const int* __restrict__ request_of,
                 const int* __restrict__ cu_q, const int* __restrict__ state_slots, int num_slots, int inner, int taps,
                 T* __restrict__ out, unsigned* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = request_of[t];
  const int first = cu_q[b], slot = state_slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
    return;
  }
  const float* tail = state + (int64_t)slot * state_stride + tail_offset;          // [taps - 1, inner]
  const int back = t - first;                                                       // tokens of the portion before this one
  for (int c = threadIdx.x; c < inner; c += blockDim.x) {
    float acc = conv_b != nullptr ? load_flex(conv_b, w_f32, c) : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int ago = taps - 1 - j;                                                 // tap j reads the input `ago` tokens back
      float u;
      if (ago <= back) u = to_f32(xz[(int64_t)(t - ago) * xz_stride + c]);
      else u = tail[(int64_t)(taps - 1 - (ago - back)) * inner + c];                // the tail's last row is the newest
      acc = fmaf(load_flex(conv_w, w_f32, (int64_t)c * taps + j), u, acc);
    }
    out[(int64_t)t * inner + c] = from_f32<T>(silu_f(acc));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
scan_tail_kernel(const T* __restrict__ xz, int64_t xz_stride, float* state, int64_t state_stride, int64_t tail_offset,
                 const int* __restrict__ cu_q, const int* __restrict__ state_slots, int num_slots, int inner, int taps) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int first = cu_q[b], n = cu_q[b + 1] - first, slot = state_slots[b];
  if (slot < 0 || slot >= num_slots || n <= 0) return;
  float* tail = state + (int64_t)slot * state_stride + tail_offset;
  const int rows = taps - 1;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < inner; c += gridDim.x * blockDim.x) {
    // row k of the new tail is the input rows - k tokens before the end of (old tail ++ portion);
    // rows are rewritten in ascending order and a row only ever reads rows above itself
    for (int k = 0; k < rows; ++k) {
      const int idx = n - (rows - k);                                               // index into the portion
      tail[(int64_t)k * inner + c] = idx >= 0 ? to_f32(xz[(int64_t)(first + idx) * xz_stride + c])
                                              : tail[(int64_t)(k + n) * inner + c];
    }
  }
}

constexpr int SCAN_CHANNELS = 32;      // channels of a block
constexpr int MAX_PER_LANE = 16;       // states a lane keeps in registers

// LANES lanes share a channel; lane r keeps states r, r + LANES, ...
template <typename T, int LANES>
__global__ void __launch_bounds__(SCAN_CHANNELS * LANES)
scan_run_kernel(const T* __restrict__ x, const float* __restrict__ dtp, const void* __restrict__ dt_bias,
                const float* __restrict__ bc, const void* __restrict__ a_log, const void* __restrict__ d_skip, int w_f32,
                const T* __restrict__ z, int64_t z_stride, float* state, int64_t state_stride, const int* __restrict__ cu_q,
                const int* __restrict__ state_slots, int num_slots, int inner, int N, T* __restrict__ y, unsigned* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int first = cu_q[b], count = cu_q[b + 1] - first, slot = state_slots[b];
  if (count <= 0) return;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
    return;
  }
  const int c = blockIdx.x * SCAN_CHANNELS + threadIdx.x / LANES, r = threadIdx.x % LANES;
  const bool live = c < inner;
  const int cc = live ? c : inner - 1;                      // idle threads follow a real channel and store nothing
  float* S = state + (int64_t)slot * state_stride + (int64_t)cc * N;
  float s[MAX_PER_LANE], a[MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int n = r + i * LANES;
    s[i] = n < N ? S[n] : 0.f;
    a[i] = n < N ? -expf(load_flex(a_log, w_f32, (int64_t)cc * N + n)) : 0.f;
  }
  const float bias = dt_bias != nullptr ? load_flex(dt_bias, w_f32, cc) : 0.f;
  const float skip = d_skip != nullptr ? load_flex(d_skip, w_f32, cc) : 0.f;
  float xv = to_f32(x[(int64_t)first * inner + cc]), dv = dtp[(int64_t)first * inner + cc];
  float zv = to_f32(z[(int64_t)first * z_stride + cc]);
  for (int i = 0; i < count; ++i) {
    const int t = first + i;
    const float xc = xv, zc = zv, dt = softplus_f(dv + bias);
    if (i + 1 < count) {
      xv = to_f32(x[(int64_t)(t + 1) * inner + cc]);
      dv = dtp[(int64_t)(t + 1) * inner + cc];
      zv = to_f32(z[(int64_t)(t + 1) * z_stride + cc]);
    }
    const float* B = bc + (int64_t)t * 2 * N;
    const float* C = B + N;
    const float dx = dt * xc;
    float part = 0.f;
#pragma unroll
    for (int k = 0; k < MAX_PER_LANE; ++k) {
      const int n = r + k * LANES;
      if (n < N) {
        s[k] = fmaf(expf(dt * a[k]), s[k], dx * B[n]);
        part = fmaf(s[k], C[n], part);
      }
    }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (live && r == 0) y[(int64_t)t * inner + c] = from_f32<T>((part + skip * xc) * silu_f(zc));
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int n = r + i * LANES;
      if (n < N) S[n] = s[i];
    }
  }
}

}  // namespace

// xz [tokens, xz_stride] holds the convolution's inputs in its first `inner` columns; out [tokens, inner].
// The state slot's tail [taps - 1, inner] starts tail_offset floats into the slot. Two launches
// when taps > 1.
VOSTI_API int vosti_scan_conv(const void* xz, int64_t xz_stride, const void* conv_w, const void* conv_b, int w_f32, float* state,
                              int64_t state_stride, int64_t tail_offset, const int* request_of, const int* cu_q,
                              const int* state_slots, int num_slots, int requests, int tokens, int inner, int taps, void* out,
                              int is_f32, unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && requests >= 0 && inner > 0 && taps >= 1 && taps <= 64, "scan_conv: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  if (is_f32)
    vosti_launch(scan_conv_kernel<float>, dim3(tokens), dim3(256), 0, stream, (const float*)xz, xz_stride, conv_w, conv_b, w_f32,
                 (const float*)state, state_stride, tail_offset, request_of, cu_q, state_slots, num_slots, inner, taps,
                 (float*)out, status);
  else
    vosti_launch(scan_conv_kernel<bf16>, dim3(tokens), dim3(256), 0, stream, (const bf16*)xz, xz_stride, conv_w, conv_b, w_f32,
                 (const float*)state, state_stride, tail_offset, request_of, cu_q, state_slots, num_slots, inner, taps,
                 (bf16*)out, status);
  if (taps > 1) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { vosti_set_error("%s", cudaGetErrorString(e)); return (int)e; }
    const int across = (inner + 255) / 256 < 64 ? (inner + 255) / 256 : 64;
    if (is_f32)
      vosti_launch(scan_tail_kernel<float>, dim3(across, requests), dim3(256), 0, stream, (const float*)xz, xz_stride, state,
                   state_stride, tail_offset, cu_q, state_slots, num_slots, inner, taps);
    else
      vosti_launch(scan_tail_kernel<bf16>, dim3(across, requests), dim3(256), 0, stream, (const bf16*)xz, xz_stride, state,
                   state_stride, tail_offset, cu_q, state_slots, num_slots, inner, taps);
  }
  VOSTI_LAUNCH_CHECK();
}

// x [tokens, inner] (after the convolution), dtp float32 [tokens, inner], bc float32 [tokens, 2 N] = B | C,
// z [tokens, z_stride] (its first `inner` columns), y [tokens, inner]; a_log [inner, N], dt_bias and
// d_skip [inner] share a type. The state S [inner, N] is the start of the slot.
VOSTI_API int vosti_scan_run(const void* x, const float* dtp, const void* dt_bias, const float* bc, const void* a_log,
                             const void* d_skip, int w_f32, const void* z, int64_t z_stride, float* state,
                             int64_t state_stride, const int* cu_q, const int* state_slots, int num_slots, int requests,
                             int inner, int N, void* y, int is_f32, unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(requests >= 0 && inner > 0 && N > 0 && N <= 8 * MAX_PER_LANE, "scan_run: bad sizes inner=%d states=%d (at most %d)",
                inner, N, 8 * MAX_PER_LANE);
  VOSTI_REQUIRE(requests <= 65535, "scan_run: too many requests for one launch");
  if (requests == 0) return VOSTI_OK;
  const dim3 grid((inner + SCAN_CHANNELS - 1) / SCAN_CHANNELS, requests);
  const int lanes = N <= 4 ? 1 : N <= 8 ? 2 : N <= 32 ? 4 : 8;       // 4 to 8 states a lane at the usual sizes
#define VOSTI_SCAN(TT, L)                                                                                               \
  vosti_launch(scan_run_kernel<TT, L>, grid, dim3(SCAN_CHANNELS * L), 0, stream, (const TT*)x, dtp, dt_bias, bc, a_log, d_skip, \
               w_f32, (const TT*)z, z_stride, state, state_stride, cu_q, state_slots, num_slots, inner, N, (TT*)y, status)
  if (is_f32) {
    if (lanes == 1) VOSTI_SCAN(float, 1); else if (lanes == 2) VOSTI_SCAN(float, 2); else if (lanes == 4) VOSTI_SCAN(float, 4); else VOSTI_SCAN(float, 8);
  } else {
    if (lanes == 1) VOSTI_SCAN(bf16, 1); else if (lanes == 2) VOSTI_SCAN(bf16, 2); else if (lanes == 4) VOSTI_SCAN(bf16, 4); else VOSTI_SCAN(bf16, 8);
  }
#undef VOSTI_SCAN
  VOSTI_LAUNCH_CHECK();
}
