// Mixture of experts: the router's choice and what it costs to apply it.
//
// moe_route: per token, the `top` experts with the largest float32 router logits (the lowest
// index wins a tie) and their weights: the softmax over the chosen logits only, or (`over_all`)
// the softmax over all experts, of which the chosen ones' scores are divided by their sum (plus
// 1e-20); either way times a constant `scale`. It writes the
// choice twice: as lists (expert ids and weights, [tokens, top]) and as a dense float32 matrix
// [tokens, experts] that is zero where an expert was not chosen.
//
// moe_router_scored: another way to choose (route_row_scored): softmax scores over all routed rows,
// the choice by score + correction inside the best groups of neighbouring rows, rows at the end
// that stand for experts returning their input, and one more router row whose sigmoid gates a
// shared expert. moe_identity adds the input-returning experts' share of the input.
//
// moe_scale: multiplies each expert's slice of the stacked activation [tokens, experts * ff] by
// the token's weight for that expert (zero for experts it did not choose), after an optional
// activation of its own (the exact GELU, for experts without a gate), so that one product
// with the experts' down projections side by side, [width, experts * ff], is the weighted sum
// of the chosen experts' outputs.
//
// For long portions the stacked product would compute every expert for every token. There the
// (token, pick) pairs are sorted by expert instead (moe_group: one block counts, scans and
// places them, so the order inside an expert's run is by pair index and the same every time),
// every expert multiplies its own run of gathered rows, and moe_combine adds a token's picks in
// the order of its picks: out[t] = sum_k w[t, k] * y[where[t, k]].
#include "common.cuh"

namespace {

// One warp: the choice for token t from its row of logits (global or shared memory).
__device__ __forceinline__ void route_row(const float* row, int t, int experts, int top, int* __restrict__ chosen,
                                          float* __restrict__ weights, float* __restrict__ dense, int over_all, float scale) {
  const int lane = threadIdx.x & 31;
  for (int e = lane; e < experts; e += 32) dense[(int64_t)t * experts + e] = 0.f;
  float first = 0.f, total = 0.f;
  unsigned long long taken_low = 0;     // experts 0..63 this lane already gave away (bit e / 32 of its share)
  for (int r = 0; r < top; ++r) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane, n = 0; e < experts; e += 32, ++n) {
      const bool taken = n < 64 ? (taken_low >> n) & 1ull : false;
      const float v = row[e];
      if (!taken && (v > best || (v == best && e < best_e))) { best = v; best_e = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    if (best_e != 0x7fffffff && (best_e & 31) == lane) taken_low |= 1ull << (best_e >> 5);
    if (r == 0) first = best;
    const float p = expf(best - first);        // the first pick is the largest logit
    total += p;
    if (lane == 0) {
      chosen[(int64_t)t * top + r] = best_e;
      weights[(int64_t)t * top + r] = p;
    }
  }
  __syncwarp();
  float inv = 1.f / total;
  if (over_all) {
    // scores over all experts: exp(z - max) / Z; the chosen ones' sum is total / Z
    float z = 0.f;
    for (int e = lane; e < experts; e += 32) z += expf(row[e] - first);
    z = warp_sum(z);
    inv = (1.f / z) / (total / z + 1e-20f);
  }
  inv *= scale;
  if (lane == 0)
    for (int r = 0; r < top; ++r) {
      const float w = weights[(int64_t)t * top + r] * inv;
      weights[(int64_t)t * top + r] = w;
      dense[(int64_t)t * experts + chosen[(int64_t)t * top + r]] = w;
    }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int tokens, int experts, int top, int* __restrict__ chosen,
                 float* __restrict__ weights, float* __restrict__ dense, int over_all, float scale) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  route_row(logits + (int64_t)t * experts, t, experts, top, chosen, weights, dense, over_all, scale);
}

// The router's product and the choice in one kernel, one block per token: the token's row goes to
// shared memory as float32, every warp makes the logits of its experts (a lane's multiply-add
// chain over k = lane, lane + 32, ..., then the warp's fixed tree: the order depends on k alone),
// and the first warp chooses. The router's matrix is float32 [experts, k].
// The token's row to shared memory as float32, then the logits of `rows` router rows into lg (and,
// if asked for, into `logits`): every warp takes the rows warp, warp + nwarps, ...
__device__ __forceinline__ void router_logits(const void* __restrict__ x, int x_f32, const float* __restrict__ router, int rows,
                                              int k, int t, float* xs, float* lg, float* __restrict__ logits) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < k; i += blockDim.x) xs[i] = load_flex(x, x_f32, (int64_t)t * k + i);
  __syncthreads();
  const int nwarps = blockDim.x >> 5;
  for (int e = warp; e < rows; e += nwarps) {
    const float* w = router + (int64_t)e * k;
    float acc = 0.f;
    if (k % 4 == 0) {
      // 16-byte words, four of them in flight: a lane's chain runs over the words lane, lane + 32, ...
      float part[4] = {0.f, 0.f, 0.f, 0.f};
      const float4* w4 = reinterpret_cast<const float4*>(w);
      const float4* x4 = reinterpret_cast<const float4*>(xs);
#pragma unroll 4
      for (int i = lane; i < k / 4; i += 32) {
        const float4 a = x4[i], b = w4[i];
        part[0] = fmaf(a.x, b.x, part[0]);
        part[1] = fmaf(a.y, b.y, part[1]);
        part[2] = fmaf(a.z, b.z, part[2]);
        part[3] = fmaf(a.w, b.w, part[3]);
      }
      acc = (part[0] + part[1]) + (part[2] + part[3]);
    } else {
      for (int i = lane; i < k; i += 32) acc = fmaf(xs[i], w[i], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      lg[e] = acc;
      if (logits != nullptr) logits[(int64_t)t * rows + e] = acc;
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(256)
moe_router_kernel(const void* __restrict__ x, int x_f32, const float* __restrict__ router, int experts, int k, int top,
                  int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ dense, float* __restrict__ logits,
                  int over_all, float scale) {
  extern __shared__ __align__(16) float router_smem[];         // [k] the token's row, then [experts] its logits
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  float* lg = router_smem + k;
  router_logits(x, x_f32, router, experts, k, t, router_smem, lg, logits);
  if ((threadIdx.x >> 5) == 0) route_row(lg, t, experts, top, chosen, weights, dense, over_all, scale);
}

// The largest value among v[i], i in [0, n), with skip[i] == 0 (skip may be null), and its index: the lowest
// index wins a tie; n = 0 or nothing left: (-inf, 0x7fffffff). One warp.
__device__ __forceinline__ void warp_argmax(const float* v, const int* skip, int n, float& best, int& best_i) {
  const int lane = threadIdx.x & 31;
  best = -INFINITY;
  best_i = 0x7fffffff;
  for (int i = lane; i < n; i += 32) {
    if (skip != nullptr && skip[i]) continue;
    const float x = v[i];
    if (x > best || (x == best && i < best_i && x != -INFINITY)) { best = x; best_i = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
}

// Choice by corrected scores inside the best groups. `routed` router rows take part: the first
// `routed - identity` are experts with matrices, the last `identity` return their input. Scores are
// s = softmax(logits) over all routed rows; a row is chosen by s + correction (correction null: by
// s); with `groups` > 1 the rows form that many equal groups of neighbours, a group's score is its
// largest choice score, and only rows of the `keep` best groups can be chosen (the others count as
// minus infinity). The weights are the chosen rows' s divided by their sum + 1e-20, times `scale`.
// Written: chosen and weights [tokens, top]; dense [tokens, dense_cols], zero but for the chosen
// experts' weights (an identity expert has no column); ident [tokens], the sum of the chosen identity
// experts' weights; and, with a gate row (the router's row number `routed`), its sigmoid in column
// routed - identity of dense. One warp; lg holds the logits, sc / ch / gs / taken / picks are scratch.
__device__ __forceinline__ void route_row_scored(const float* lg, int t, int routed, int identity, int top, const float* __restrict__ correction,
                                                 int groups, int keep, int gate_rows, float scale, float* sc, float* ch, float* gs,
                                                 int* taken, int* picks, int* __restrict__ chosen, float* __restrict__ weights,
                                                 float* __restrict__ dense, float* __restrict__ ident, int dense_cols) {
  const int lane = threadIdx.x & 31;
  const int experts = routed - identity;
  float top_logit = -INFINITY;
  for (int e = lane; e < routed; e += 32) top_logit = fmaxf(top_logit, lg[e]);
  top_logit = warp_max(top_logit);
  float z = 0.f;
  for (int e = lane; e < routed; e += 32) {
    const float p = expf(lg[e] - top_logit);
    sc[e] = p;
    z += p;
  }
  z = warp_sum(z);
  const float inv_z = 1.f / z;
  for (int e = lane; e < routed; e += 32) {
    const float s = sc[e] * inv_z;
    sc[e] = s;
    ch[e] = correction != nullptr ? s + correction[e] : s;
  }
  for (int c = lane; c < dense_cols; c += 32) dense[(int64_t)t * dense_cols + c] = 0.f;
  __syncwarp();
  if (groups > 1) {
    const int per = routed / groups;
    for (int g = lane; g < groups; g += 32) {
      float m = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, ch[e]);
      gs[g] = m;
      taken[g] = 0;
    }
    __syncwarp();
    for (int r = 0; r < keep; ++r) {
      float best;
      int best_g;
      warp_argmax(gs, taken, groups, best, best_g);
      if (lane == 0 && best_g != 0x7fffffff) taken[best_g] = 1;
      __syncwarp();
    }
    for (int e = lane; e < routed; e += 32)
      if (!taken[e / per]) ch[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int r = 0; r < top; ++r) {
    float best;
    int best_e;
    warp_argmax(ch, nullptr, routed, best, best_e);
    if (best_e == 0x7fffffff) best_e = 0;               // nothing left to choose from: a malformed router (top > rows allowed)
    __syncwarp();
    if (lane == 0) {
      ch[best_e] = -INFINITY;
      picks[r] = best_e;
    }
    total += sc[best_e];
    __syncwarp();
  }
  // a lane a pick: ids, weights, the dense row; the identity experts' share summed over the lanes
  const float inv = scale / (total + 1e-20f);
  float own = 0.f;
  for (int r = lane; r < top; r += 32) {
    const int e = picks[r];
    const float w = sc[e] * inv;
    chosen[(int64_t)t * top + r] = e;
    weights[(int64_t)t * top + r] = w;
    if (e < experts) dense[(int64_t)t * dense_cols + e] = w;
    else own += w;
  }
  own = warp_sum(own);
  if (lane == 0) {
    if (ident != nullptr) ident[t] = own;
    if (gate_rows) dense[(int64_t)t * dense_cols + experts] = 1.f / (1.f + expf(-lg[routed]));
  }
}

// Router product and scored choice in one kernel, one block per token (see route_row_scored). The
// router's matrix is float32 [routed + gate_rows, k].
__global__ void __launch_bounds__(1024)
moe_router_scored_kernel(const void* __restrict__ x, int x_f32, const float* __restrict__ router, int routed, int identity, int k,
                         int top, const float* __restrict__ correction, int groups, int keep, int gate_rows, float scale,
                         int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ dense, float* __restrict__ ident,
                         int dense_cols, float* __restrict__ logits) {
  extern __shared__ __align__(16) float router_smem[];   // [k] row, [rows] logits, [routed] scores, [routed] choice scores, [groups] x 2, [top] picks
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, rows = routed + gate_rows;
  const int kpad = (k + 3) & ~3;
  float* lg = router_smem + kpad;
  float* sc = lg + rows;
  float* ch = sc + routed;
  float* gs = ch + routed;
  int* taken = reinterpret_cast<int*>(gs + groups);
  int* picks = taken + groups;
  router_logits(x, x_f32, router, rows, k, t, router_smem, lg, logits);
  if ((threadIdx.x >> 5) == 0)
    route_row_scored(lg, t, routed, identity, top, correction, groups, keep, gate_rows, scale, sc, ch, gs, taken, picks, chosen, weights,
                     dense, ident, dense_cols);
}

// `dense` null: the activation alone.
// `gelu`: 0 no activation, 1 the exact GELU, 2 the square of relu. `tail` > 0: after the experts' slices
// the row holds one more slice of `tail` columns (a shared expert of another width), whose weight is
// column `experts` of dense, which then has experts + 1 columns.
__device__ __forceinline__ float moe_activation(float x, int mode) {
  if (mode == 1) return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
  if (mode == 2) { x = fmaxf(x, 0.f); return x * x; }
  return x;
}

template <typename T>
__global__ void moe_scale_kernel(T* __restrict__ act, const float* __restrict__ dense, int64_t tokens, int experts, int ff,
                                 int gelu, int tail) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t width = (int64_t)experts * ff + tail, n = tokens * width;
  const int cols = experts + (tail > 0 ? 1 : 0);
  if (sizeof(T) == 2 && ff % 8 == 0 && tail % 8 == 0 && (reinterpret_cast<uintptr_t>(act) & 15) == 0) {
    // 16-byte words: eight elements of one expert's slice
    const int64_t words = n / 8, per_row = width / 8;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (int64_t)gridDim.x * blockDim.x) {
      const int64_t t = w / per_row;
      const int64_t c = (w - t * per_row) * 8;
      const int e = c < (int64_t)experts * ff ? (int)(c / ff) : experts;
      const float by = dense != nullptr ? dense[t * cols + e] : 1.f;
      uint4 raw = reinterpret_cast<uint4*>(act)[w];
      __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(p[k]);
        float a = moe_activation(f.x, gelu), b = moe_activation(f.y, gelu);
        if (dense != nullptr) { a *= by; b *= by; }
        p[k] = __floats2bfloat162_rn(a, b);
      }
      reinterpret_cast<uint4*>(act)[w] = raw;
    }
    return;
  }
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / width;
    const int64_t c = i - t * width;
    const int e = c < (int64_t)experts * ff ? (int)(c / ff) : experts;
    float x = moe_activation(to_f32(act[i]), gelu);
    if (dense != nullptr) x *= dense[t * cols + e];
    act[i] = from_f32<T>(x);
  }
}

// y[t, :] += coeff[t] * x[t, :] (y float32; x float32 or bfloat16): what experts that return their
// input add to a mixture's output.
__global__ void __launch_bounds__(256)
moe_identity_kernel(float* __restrict__ y, const float* __restrict__ coeff, const void* __restrict__ x, int x_f32, int width) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  const float c = coeff[blockIdx.x];
  if (c == 0.f) return;
  for (int i = threadIdx.x; i < width; i += blockDim.x) y[base + i] = fmaf(c, load_flex(x, x_f32, base + i), y[base + i]);
}

// One block. chosen: [pairs] expert of every (token, pick) pair, pair = token * top + pick.
// offsets [experts + 1]: where each expert's run starts in the sorted order; rows [pairs]: the
// token of the pair at each sorted place; where [pairs]: the sorted place of each pair.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ chosen, int pairs, int top, int experts, int* __restrict__ offsets,
                 int* __restrict__ rows, int* __restrict__ where) {
  extern __shared__ int counts[];           // [experts + 1]
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = chosen[i];
    if (e >= 0 && e < experts) atomicAdd(&counts[e + 1], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int e = 0; e < experts; ++e) counts[e + 1] += counts[e];
    for (int e = 0; e <= experts; ++e) offsets[e] = counts[e];
  }
  __syncthreads();
  // a pair's place: its expert's start plus the number of earlier pairs of the same expert.
  // One warp per expert walks the pairs in order, so the placement never varies.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int e = warp; e < experts; e += nwarps) {
    int at = counts[e];
    for (int i0 = 0; i0 < pairs; i0 += 32) {
      const int i = i0 + lane;
      const bool mine = i < pairs && chosen[i] == e;
      const unsigned ballot = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int place = at + __popc(ballot & ((1u << lane) - 1u));
        rows[place] = i / top;
        where[i] = place;
      }
      at += __popc(ballot);
    }
  }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ where, const float* __restrict__ weights,
                   float* __restrict__ out, int top, int width) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(weights[(int64_t)t * top + k], y[(int64_t)where[(int64_t)t * top + k] * width + c], acc);
    out[(int64_t)t * width + c] = acc;
  }
}

}  // namespace

VOSTI_API int vosti_moe_group(const int* chosen, int tokens, int top, int experts, int* offsets, int* rows, int* where,
                              cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && top > 0 && experts > 0 && experts <= 8192, "moe_group: bad sizes");
  VOSTI_REQUIRE((int64_t)tokens * top < (int64_t)1 << 30, "moe_group: too many pairs");
  vosti_launch(moe_group_kernel, dim3(1), dim3(1024), (size_t)(experts + 1) * sizeof(int), stream, chosen, tokens * top, top,
               experts, offsets, rows, where);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_moe_combine(const float* y, const int* where, const float* weights, float* out, int tokens, int top,
                                int width, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && top > 0 && width > 0, "moe_combine: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  vosti_launch(moe_combine_kernel, dim3(tokens), dim3(256), 0, stream, y, where, weights, out, top, width);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_moe_route(const float* logits, int tokens, int experts, int top, int* chosen, float* weights,
                              float* dense, int over_all, float scale, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts, "moe_route: bad sizes experts=%d top=%d", experts, top);
  VOSTI_REQUIRE(experts <= 2048, "moe_route: %d experts (at most 2048 are taken)", experts);
  if (tokens == 0) return VOSTI_OK;
  vosti_launch(moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, stream, logits, tokens, experts, top, chosen, weights, dense, over_all, scale);
  VOSTI_LAUNCH_CHECK();
}

static int moe_scale_launch(void* act, const float* dense, int tokens, int experts, int ff, int is_f32, int gelu, int tail,
                            cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && experts >= 0 && ff > 0 && tail >= 0 && (experts > 0 || tail > 0) && gelu >= 0 && gelu <= 2,
                "moe_scale: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int64_t n = (int64_t)tokens * ((int64_t)experts * ff + tail);
  const int64_t items = (!is_f32 && ff % 8 == 0 && tail % 8 == 0) ? n / 8 : n;      // 16-byte words where the slices allow them
  const int blocks = (int)((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
  if (is_f32) vosti_launch(moe_scale_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)act, dense, (int64_t)tokens, experts, ff, gelu, tail);
  else vosti_launch(moe_scale_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)act, dense, (int64_t)tokens, experts, ff, gelu, tail);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_moe_scale(void* act, const float* dense, int tokens, int experts, int ff, int is_f32, int gelu,
                              cudaStream_t stream) {
  return moe_scale_launch(act, dense, tokens, experts, ff, is_f32, gelu, 0, stream);
}

// The same with an activation mode (0 none, 1 exact GELU, 2 squared relu) and a tail slice of `tail`
// columns whose weight is dense's last column (dense: [tokens, experts + (tail > 0)]).
VOSTI_API int vosti_moe_scale_tail(void* act, const float* dense, int tokens, int experts, int ff, int tail, int is_f32,
                                   int activation, cudaStream_t stream) {
  return moe_scale_launch(act, dense, tokens, experts, ff, is_f32, activation, tail, stream);
}

VOSTI_API int vosti_moe_identity(float* y, const float* coeff, const void* x, int x_f32, int tokens, int width, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && width > 0, "moe_identity: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  vosti_launch(moe_identity_kernel, dim3(tokens), dim3(256), 0, stream, y, coeff, x, x_f32, width);
  VOSTI_LAUNCH_CHECK();
}

// x [tokens, k] float32 or bfloat16; router float32 [routed + gate_rows, k]; correction float32 [routed]
// or null; dense float32 [tokens, routed - identity + gate_rows]; ident float32 [tokens] (or null when
// there are no identity experts); `logits` (optional) float32 [tokens, routed + gate_rows].
VOSTI_API int vosti_moe_router_scored(const void* x, int x_f32, const float* router, int tokens, int routed, int identity, int k,
                                      int top, const float* correction, int groups, int keep, int gate_rows, float scale,
                                      int* chosen, float* weights, float* dense, float* ident, float* logits,
                                      cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && routed > 0 && identity >= 0 && identity <= routed && k > 0 && (gate_rows == 0 || gate_rows == 1),
                "moe_router: bad sizes routed=%d identity=%d", routed, identity);
  VOSTI_REQUIRE(routed <= 2048, "moe_router: %d experts (at most 2048 are taken)", routed);
  VOSTI_REQUIRE(groups >= 1 && routed % groups == 0 && keep >= 1 && keep <= groups, "moe_router: %d groups of which %d are kept do not divide %d experts", groups, keep, routed);
  VOSTI_REQUIRE(top > 0 && top <= (routed / groups) * keep, "moe_router: top %d exceeds the experts of the kept groups", top);
  VOSTI_REQUIRE(identity == 0 || ident != nullptr, "moe_router: identity experts need their output");
  const size_t smem = (size_t)(((k + 3) & ~3) + routed + gate_rows + 2 * routed + 2 * groups + top) * sizeof(float);
  VOSTI_REQUIRE(smem <= 200 * 1024, "moe_router: a row of %d elements does not fit shared memory", k);
  if (tokens == 0) return VOSTI_OK;
  {
    static bool configured = false;       // once, to the most a launch may ask for
    if (!configured) {
      cudaFuncSetAttribute(moe_router_scored_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      configured = true;
    }
  }
  // a warp a router row, so that all rows' products run side by side
  const int rows = routed + gate_rows;
  const int threads = rows >= 32 ? 1024 : (rows > 4 ? rows * 32 : 128);
  vosti_launch(moe_router_scored_kernel, dim3(tokens), dim3(threads), smem, stream, x, x_f32, router, routed, identity, k, top,
               correction, groups, keep, gate_rows, scale, chosen, weights, dense, ident, routed - identity + gate_rows, logits);
  VOSTI_LAUNCH_CHECK();
}

// x [tokens, k] float32 or bfloat16; router float32 [experts, k]; `logits` (optional) receives the
// float32 logits [tokens, experts].
VOSTI_API int vosti_moe_router(const void* x, int x_f32, const float* router, int tokens, int experts, int k, int top,
                               int* chosen, float* weights, float* dense, float* logits, int over_all, float scale,
                               cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts && k > 0, "moe_router: bad sizes experts=%d top=%d", experts, top);
  VOSTI_REQUIRE(experts <= 2048, "moe_router: %d experts (at most 2048 are taken)", experts);
  const size_t smem = (size_t)(k + experts) * sizeof(float);
  VOSTI_REQUIRE(smem <= 200 * 1024, "moe_router: a row of %d elements does not fit shared memory", k);
  if (tokens == 0) return VOSTI_OK;
  {
    static bool configured = false;       // once, to the most a launch may ask for
    if (!configured) {
      cudaFuncSetAttribute(moe_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      configured = true;
    }
  }
  vosti_launch(moe_router_kernel, dim3(tokens), dim3(experts > 4 ? 256 : 128), smem, stream, x, x_f32, router, experts, k, top, chosen, weights,
               dense, logits, over_all, scale);
  VOSTI_LAUNCH_CHECK();
}
