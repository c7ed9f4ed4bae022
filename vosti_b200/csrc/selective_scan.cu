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
//   scan_run    the recurrence: a block per (request, 32 channels, chunk of tokens), LANES lanes share a
//               channel and split its states; tokens in order. A portion of several chunks takes three
//               launches (each chunk from zero, the chunks' start states, each chunk from its start).
//               Everything after the projections is float32.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// A thread takes one channel (neighbouring threads neighbouring channels) and `per_block` tokens one
// after the other. With up to 8 taps the taps' weights and the last inputs stay in registers: a token
// costs one load; the window is filled anew at the block's first token and where a request starts.
constexpr int CONV_WINDOW = 8;

template <typename T>
__global__ void __launch_bounds__(256)
scan_conv_kernel(const T* __restrict__ xz, int64_t xz_stride, const void* __restrict__ conv_w, const void* __restrict__ conv_b,
                 int w_f32, const float* state, int64_t state_stride, int64_t tail_offset, const int* __restrict__ request_of,
                 const int* __restrict__ cu_q, const int* __restrict__ state_slots, int num_slots, int inner, int taps,
                 int tokens, int per_block, T* __restrict__ out, unsigned* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t_begin = blockIdx.y * per_block, t_end = min(tokens, t_begin + per_block);
  const bool live = c < inner;
  const float bias = live && conv_b != nullptr ? load_flex(conv_b, w_f32, c) : 0.f;
  // the input `ago` tokens before token t of request b (portion starting at `first`, state in `tail`)
  auto input = [&](int t, int ago, int first, const float* tail) {
    const int back = t - first;
    return ago <= back ? to_f32(xz[(int64_t)(t - ago) * xz_stride + c])
                       : tail[(int64_t)(taps - 1 - (ago - back)) * inner + c];           // the tail's last row is the newest
  };
  int b = -1, first = 0, next_first = 0;
  const float* tail = nullptr;
  bool usable = false;
  if (taps <= CONV_WINDOW) {
    float w[CONV_WINDOW], win[CONV_WINDOW];          // right-aligned: index CONV_WINDOW - 1 - k is k tokens ago
#pragma unroll
    for (int k = 0; k < CONV_WINDOW; ++k) {
      w[CONV_WINDOW - 1 - k] = live && k < taps ? load_flex(conv_w, w_f32, (int64_t)c * taps + taps - 1 - k) : 0.f;
      win[k] = 0.f;
    }
    for (int t = t_begin; t < t_end; ++t) {
      const bool fresh = b < 0 || t >= next_first;
      if (fresh) {
        b = request_of[t];
        first = cu_q[b];
        next_first = cu_q[b + 1];
        const int slot = state_slots[b];
        usable = slot >= 0 && slot < num_slots;
        if (!usable && threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
        tail = state + (int64_t)(usable ? slot : 0) * state_stride + tail_offset;        // [taps - 1, inner]
      }
      if (!usable || !live) continue;
      if (fresh) {
#pragma unroll
        for (int k = 1; k < CONV_WINDOW; ++k) win[CONV_WINDOW - 1 - k] = k < taps ? input(t, k, first, tail) : 0.f;
      } else {
#pragma unroll
        for (int k = CONV_WINDOW - 1; k >= 1; --k) win[CONV_WINDOW - 1 - k] = win[CONV_WINDOW - k];
      }
      win[CONV_WINDOW - 1] = to_f32(xz[(int64_t)t * xz_stride + c]);
      // oldest tap first, as in the loop over the taps below
      float acc = bias;
#pragma unroll
      for (int k = CONV_WINDOW - 1; k >= 0; --k)
        if (k < taps) acc = fmaf(w[CONV_WINDOW - 1 - k], win[CONV_WINDOW - 1 - k], acc);
      out[(int64_t)t * inner + c] = from_f32<T>(silu_f(acc));
    }
    return;
  }
  for (int t = t_begin; t < t_end; ++t) {
    if (b < 0 || t >= next_first) {
      b = request_of[t];
      first = cu_q[b];
      next_first = cu_q[b + 1];
      const int slot = state_slots[b];
      usable = slot >= 0 && slot < num_slots;
      if (!usable && threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
      tail = state + (int64_t)(usable ? slot : 0) * state_stride + tail_offset;
    }
    if (!usable || !live) continue;
    float acc = bias;
    for (int j = 0; j < taps; ++j)                                                      // tap j reads the input taps - 1 - j tokens back
      acc = fmaf(load_flex(conv_w, w_f32, (int64_t)c * taps + j), input(t, taps - 1 - j, first, tail), acc);
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

// One block runs at most `chunk` tokens of one request for 32 channels; LANES lanes share a channel
// and lane r keeps its states r, r + LANES, ... (PER of them at most) in registers. The block first
// brings its tokens' inputs into shared memory with the per-(token, channel) functions already
// applied (softplus of the step size, silu of the gate), so that the loop over tokens holds only
// the recurrence; the gated read-outs collect in shared memory and leave in rows.
//
// A portion longer than `chunk` is cut into chunks that run side by side. The recurrence is linear in
// the state, S_end = P S_start + L with P = exp(A * sum of the chunk's step sizes) and L the state
// the chunk reaches from zero. LOCAL = true computes L and the sum for every chunk but the last;
// scan_carry_kernel then walks a request's chunks and leaves every chunk's start state; LOCAL = false
// runs each chunk from its start state and writes the read-outs, the last chunk also the slot.
// A portion of one chunk takes the slot's state directly (one launch).
//
// ws [chunk slots, inner, N]: slot base(b) + k is the start state of request b's chunk k, with
// base(b) = first token of b / chunk + b (so that no two requests share a slot); ws_dt [chunk slots,
// inner] the chunks' sums of step sizes.
template <typename T, int LANES, int PER, bool LOCAL>
__global__ void __launch_bounds__(SCAN_CHANNELS * LANES)
scan_run_kernel(const T* __restrict__ x, const float* __restrict__ dtp, const void* __restrict__ dt_bias,
                const float* __restrict__ bc, const void* __restrict__ a_log, const void* __restrict__ d_skip, int w_f32,
                const T* __restrict__ z, int64_t z_stride, float* state, int64_t state_stride, const int* __restrict__ cu_q,
                const int* __restrict__ state_slots, int num_slots, int inner, int N, int chunk, float* ws, float* ws_dt,
                T* __restrict__ y, unsigned* status) {
  extern __shared__ float scan_shared[];
  float* sB = scan_shared;                                   // [chunk, 2 N]: B | C of each token
  float* sx = sB + (int64_t)chunk * 2 * N;                   // [chunk, 32]
  float* sdt = sx + chunk * SCAN_CHANNELS;                   // [chunk, 32]: softplus(step + bias)
  float* sg = sdt + chunk * SCAN_CHANNELS;                   // [chunk, 32]: silu(z), then the read-out
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y, k = blockIdx.z;
  const int first = cu_q[b], count = cu_q[b + 1] - first, slot = state_slots[b];
  const int chunks = (count + chunk - 1) / chunk;
  if (k >= (LOCAL ? chunks - 1 : chunks)) return;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0 && k == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
    return;
  }
  const int t0 = first + k * chunk, tokens = min(chunk, count - k * chunk);
  const int c0 = blockIdx.x * SCAN_CHANNELS;
  const int threads = SCAN_CHANNELS * LANES;
  for (int i = threadIdx.x; i < tokens * 2 * N; i += threads) sB[i] = bc[(int64_t)t0 * 2 * N + i];
  for (int i = threadIdx.x; i < tokens * SCAN_CHANNELS; i += threads) {
    const int t = t0 + i / SCAN_CHANNELS, ch = c0 + i % SCAN_CHANNELS;
    float xv = 0.f, dv = 0.f, gv = 0.f;
    if (ch < inner) {
      xv = to_f32(x[(int64_t)t * inner + ch]);
      dv = softplus_f(dtp[(int64_t)t * inner + ch] + (dt_bias != nullptr ? load_flex(dt_bias, w_f32, ch) : 0.f));
      if (!LOCAL) gv = silu_f(to_f32(z[(int64_t)t * z_stride + ch]));
    }
    sx[i] = xv;
    sdt[i] = dv;
    if (!LOCAL) sg[i] = gv;
  }
  const int cl = threadIdx.x / LANES, r = threadIdx.x % LANES;
  const int c = c0 + cl;
  const bool live = c < inner;
  const int cc = live ? c : inner - 1;                      // idle threads follow a real channel and store nothing
  const int64_t plane = (int64_t)inner * N;
  const int64_t base = first / chunk + b;
  float* S = state + (int64_t)slot * state_stride + (int64_t)cc * N;
  const float* start = LOCAL ? nullptr : chunks == 1 ? S : ws + (base + k) * plane + (int64_t)cc * N;
  float s[PER], a[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int n = r + i * LANES;
    s[i] = !LOCAL && n < N ? start[n] : 0.f;
    a[i] = n < N ? -expf(load_flex(a_log, w_f32, (int64_t)cc * N + n)) : 0.f;
  }
  const float skip = d_skip != nullptr ? load_flex(d_skip, w_f32, cc) : 0.f;
  __syncthreads();
  float sum = 0.f;
  for (int i = 0; i < tokens; ++i) {
    const float dt = sdt[i * SCAN_CHANNELS + cl], xc = sx[i * SCAN_CHANNELS + cl];
    const float* B = sB + (int64_t)i * 2 * N;
    const float* C = B + N;
    const float dx = dt * xc;
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int n = r + j * LANES;
      if (n < N) {
        s[j] = fmaf(expf(dt * a[j]), s[j], dx * B[n]);
        if (!LOCAL) part = fmaf(s[j], C[n], part);
      }
    }
    if (LOCAL) {
      sum += dt;
    } else {
#pragma unroll
      for (int o = LANES / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (r == 0) sg[i * SCAN_CHANNELS + cl] = (part + skip * xc) * sg[i * SCAN_CHANNELS + cl];
    }
  }
  if (live) {
    float* end = LOCAL ? ws + (base + k + 1) * plane + (int64_t)cc * N : k == chunks - 1 ? S : nullptr;
    if (end != nullptr) {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int n = r + i * LANES;
        if (n < N) end[n] = s[i];
      }
    }
    if (LOCAL && r == 0) ws_dt[(base + k) * inner + c] = sum;
  }
  if (LOCAL) return;
  __syncthreads();
  for (int i = threadIdx.x; i < tokens * SCAN_CHANNELS; i += threads) {
    const int ch = c0 + i % SCAN_CHANNELS;
    if (ch < inner) y[(int64_t)(t0 + i / SCAN_CHANNELS) * inner + ch] = from_f32<T>(sg[i]);
  }
}

// Start states of a request's chunks, one thread per (request, channel, state): chunk 0 starts from
// the slot; chunk k + 1 from exp(A * the sum of chunk k's step sizes) * (start of k) + (what chunk k reaches from zero),
// which scan_run_kernel<LOCAL> left in chunk k + 1's place.
__global__ void __launch_bounds__(256)
scan_carry_kernel(const void* __restrict__ a_log, int w_f32, const float* state, int64_t state_stride, const int* __restrict__ cu_q,
                  const int* __restrict__ state_slots, int num_slots, int inner, int N, int chunk, float* ws, const float* ws_dt) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int first = cu_q[b], count = cu_q[b + 1] - first, slot = state_slots[b];
  const int chunks = (count + chunk - 1) / chunk;
  if (chunks <= 1 || slot < 0 || slot >= num_slots) return;
  const int64_t plane = (int64_t)inner * N, base = first / chunk + b;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < plane; i += (int64_t)gridDim.x * blockDim.x) {
    const float a = -expf(load_flex(a_log, w_f32, i));
    const int c = (int)(i / N);
    float s = state[(int64_t)slot * state_stride + i];
    ws[base * plane + i] = s;
    for (int k = 0; k + 1 < chunks; ++k) {
      s = fmaf(expf(a * ws_dt[(base + k) * inner + c]), s, ws[(base + k + 1) * plane + i]);
      ws[(base + k + 1) * plane + i] = s;
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
  const int across_c = (inner + 255) / 256;
  int per_block = 1;                      // tokens a block takes: more once the grid fills the GPU several times over
  while (per_block < 16 && (int64_t)across_c * ((tokens + per_block - 1) / per_block) > 148 * 16) per_block *= 2;
  const int token_blocks = (tokens + per_block - 1) / per_block;
  VOSTI_REQUIRE(token_blocks <= 65535, "scan_conv: too many tokens for one launch");
  const dim3 grid(across_c, token_blocks);
  if (is_f32)
    vosti_launch(scan_conv_kernel<float>, grid, dim3(256), 0, stream, (const float*)xz, xz_stride, conv_w, conv_b, w_f32,
                 (const float*)state, state_stride, tail_offset, request_of, cu_q, state_slots, num_slots, inner, taps,
                 tokens, per_block, (float*)out, status);
  else
    vosti_launch(scan_conv_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)xz, xz_stride, conv_w, conv_b, w_f32,
                 (const float*)state, state_stride, tail_offset, request_of, cu_q, state_slots, num_slots, inner, taps,
                 tokens, per_block, (bf16*)out, status);
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

// Tokens a block of scan_run takes (a portion longer than this is run as chunks side by side):
// the chunk's inputs fit the shared memory every block may have without asking.
VOSTI_API int vosti_scan_chunk(int N) { return N <= 32 ? 64 : 32; }

// x [tokens, inner] (after the convolution), dtp float32 [tokens, inner], bc float32 [tokens, 2 N] = B | C,
// z [tokens, z_stride] (its first `inner` columns), y [tokens, inner]; a_log [inner, N], dt_bias and
// d_skip [inner] share a type. The state S [inner, N] is the start of the slot. When the longest
// portion exceeds vosti_scan_chunk(N) tokens, ws [tokens / chunk + requests, inner, N] and ws_dt
// [tokens / chunk + requests, inner] (float32) are needed and three kernels run instead of one.
VOSTI_API int vosti_scan_run(const void* x, const float* dtp, const void* dt_bias, const float* bc, const void* a_log,
                             const void* d_skip, int w_f32, const void* z, int64_t z_stride, float* state,
                             int64_t state_stride, const int* cu_q, const int* state_slots, int num_slots, int requests,
                             int longest, int inner, int N, float* ws, float* ws_dt, void* y, int is_f32, unsigned* status,
                             cudaStream_t stream) {
  VOSTI_REQUIRE(requests >= 0 && inner > 0 && N > 0 && N <= 128 && longest >= 0, "scan_run: bad sizes inner=%d states=%d (at most 128)",
                inner, N);
  VOSTI_REQUIRE(requests <= 65535, "scan_run: too many requests for one launch");
  if (requests == 0 || longest == 0) return VOSTI_OK;
  const int chunk = vosti_scan_chunk(N);
  const int chunks = (longest + chunk - 1) / chunk;
  VOSTI_REQUIRE(chunks <= 65535, "scan_run: a portion of %d tokens is too long for one launch", longest);
  VOSTI_REQUIRE(chunks == 1 || (ws != nullptr && ws_dt != nullptr), "scan_run: a portion of several chunks needs its workspace");
  const int groups = (inner + SCAN_CHANNELS - 1) / SCAN_CHANNELS;
  const size_t shared = (size_t)chunk * (2 * N + 3 * SCAN_CHANNELS) * sizeof(float);
  const int lanes = N <= 4 ? 1 : N <= 8 ? 2 : N <= 32 ? 4 : 8;       // 4 to 8 states a lane at the usual sizes
  const int per = (N + lanes - 1) / lanes <= 4 ? 4 : (N + lanes - 1) / lanes <= 8 ? 8 : 16;
#define VOSTI_SCAN(TT, L, P, LOCAL, GRID)                                                                                       \
  vosti_launch(scan_run_kernel<TT, L, P, LOCAL>, GRID, dim3(SCAN_CHANNELS * L), shared, stream, (const TT*)x, dtp, dt_bias, bc, a_log, \
               d_skip, w_f32, (const TT*)z, z_stride, state, state_stride, cu_q, state_slots, num_slots, inner, N, chunk, ws, \
               ws_dt, (TT*)y, status)
#define VOSTI_SCAN_SHAPE(TT, LOCAL, GRID)                                                         \
  do {                                                                                            \
    if (lanes == 1) VOSTI_SCAN(TT, 1, 4, LOCAL, GRID);                                            \
    else if (lanes == 2) VOSTI_SCAN(TT, 2, 4, LOCAL, GRID);                                       \
    else if (lanes == 4 && per == 4) VOSTI_SCAN(TT, 4, 4, LOCAL, GRID);                           \
    else if (lanes == 4) VOSTI_SCAN(TT, 4, 8, LOCAL, GRID);                                       \
    else if (per <= 8) VOSTI_SCAN(TT, 8, 8, LOCAL, GRID);                                         \
    else VOSTI_SCAN(TT, 8, 16, LOCAL, GRID);                                                      \
  } while (0)
  if (chunks > 1) {
    const dim3 grid(groups, requests, chunks - 1);
    if (is_f32) VOSTI_SCAN_SHAPE(float, true, grid); else VOSTI_SCAN_SHAPE(bf16, true, grid);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { vosti_set_error("%s", cudaGetErrorString(e)); return (int)e; }
    const int64_t plane = (int64_t)inner * N;
    const int across = (int)((plane + 255) / 256 < 1024 ? (plane + 255) / 256 : 1024);
    vosti_launch(scan_carry_kernel, dim3(across, requests), dim3(256), 0, stream, a_log, w_f32, (const float*)state, state_stride,
                 cu_q, state_slots, num_slots, inner, N, chunk, ws, (const float*)ws_dt);
    e = cudaGetLastError();
    if (e != cudaSuccess) { vosti_set_error("%s", cudaGetErrorString(e)); return (int)e; }
  }
  const dim3 grid(groups, requests, chunks);
  if (is_f32) VOSTI_SCAN_SHAPE(float, false, grid); else VOSTI_SCAN_SHAPE(bf16, false, grid);
#undef VOSTI_SCAN_SHAPE
#undef VOSTI_SCAN
  VOSTI_LAUNCH_CHECK();
}
