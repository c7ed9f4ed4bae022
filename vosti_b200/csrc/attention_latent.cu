// Latent attention: keys and values of all heads are made from one small latent vector per
// token, c [rank], and one rotated key part r [rot] that the heads share. Only c and r are
// cached (two page tensors of widths rank and rot, one "head"). With per-head matrices
// K_h [dim, rank] (unrotated keys k_h = K_h c) and V_h [vdim, rank] (values v_h = V_h c),
//
//   score_h(i, j) = (q_h . K_h c_j + qr_h . r_j) * scale = ((K_h^T q_h) . c_j + qr_h . r_j) * scale
//   o_h(i)        = sum_j p_h(i, j) V_h c_j            = V_h (sum_j p_h(i, j) c_j)
//
// so every head attends over the cached latents directly: the query is carried into the latent
// space once per token (head_project with K_h), the attention reads c and r and returns the
// weighted latent, which head_project with V_h carries back. No per-head key or value of a
// cached token is ever formed.
//
// Kernels (float32 arithmetic for both storage types):
//   latent_prep     after the q | down | gate projection, one block per token: the rotated part of
//                   every query head (the last `rot` elements of a head) is turned and written
//                   behind the place of the query's latent form; the first `rank` elements of the
//                   down projection are divided by their root mean square, weighted and stored as
//                   c; the last `rot`, turned, as r; the gates pass a sigmoid.
//   head_project    y[t, h, :] = g[t, h] * (x[t, h, :] @ M_h), M_h a strided view, on the CUDA cores.
//   latent_attend   one warp per (token, head), 32 keys at a time aligned to the absolute key index
//                   (a row's arithmetic does not depend on the cut or the batch); with few rows the
//                   keys are cut into segments and merged in order by latent_merge.
// Rotation: element i of the rotated part pairs with i + rot/2, angle = position * freq[i] in
// float32, cos and sin multiplied by `magnitude`.
#include "common.cuh"

namespace {
constexpr int WARPS = 16;            // warps of a block: the heads of one token share their keys through L1
constexpr float LOG2E = 1.4426950408889634f;

template <typename T>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const T* __restrict__ proj, int64_t proj_stride, T* __restrict__ qk, float* __restrict__ gate,
                   T* __restrict__ c_cache, T* __restrict__ r_cache, const void* __restrict__ norm_w, int norm_f32, float eps,
                   const int* __restrict__ positions, const int* __restrict__ slot_mapping, int64_t num_slots, int heads,
                   int dim, int rot, int rank, const float* __restrict__ freq, float magnitude, unsigned* status) {
  extern __shared__ float turn[];            // [rot]: cosines, then sines
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, half = rot / 2;
  const T* row = proj + (int64_t)t * proj_stride;
  const float p = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = p * freq[i];
    turn[i] = cosf(angle) * magnitude;
    turn[half + i] = sinf(angle) * magnitude;
  }
  __syncthreads();
  auto turned = [&](const T* src, int i) {          // element i of a rotated part that starts at src
    const float x = to_f32(src[i]);
    if (i < half) return x * turn[i] - to_f32(src[i + half]) * turn[half + i];
    return x * turn[i - half] + to_f32(src[i - half]) * turn[i];
  };
  const int qw = dim + rot, kw = rank + rot;
  for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
    const int h = i / rot, j = i % rot;
    qk[((int64_t)t * heads + h) * kw + rank + j] = from_f32<T>(turned(row + h * qw + dim, j));
  }
  const T* down = row + heads * qw;
  const T* graw = down + kw;
  for (int i = threadIdx.x; i < heads; i += blockDim.x) gate[(int64_t)t * heads + i] = 1.f / (1.f + expf(-to_f32(graw[i])));
  if (c_cache == nullptr) return;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f32(down[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  const int64_t slot = slot_mapping[t];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
    return;
  }
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    c_cache[slot * rank + i] = from_f32<T>(to_f32(down[i]) * inv * load_flex(norm_w, norm_f32, i));
  for (int i = threadIdx.x; i < rot; i += blockDim.x) r_cache[slot * rot + i] = from_f32<T>(turned(down + rank, i));
}

// y[t, h, o] = g[t, h] * sum_i x[t, h, i] * M[h * m_head + i * m_in + o * m_out]; a block takes 16
// tokens x 128 outputs of one head, the inner extent in pieces of 32 through shared memory.
constexpr int HP_TOKENS = 16, HP_OUT = 128, HP_IN = 32;

template <typename TX, typename TM, typename TY>
__global__ void __launch_bounds__(HP_OUT)
head_project_kernel(const TX* __restrict__ x, int64_t x_row, int64_t x_head, const TM* __restrict__ m, int64_t m_head,
                    int64_t m_in, int64_t m_out, const float* __restrict__ gate, TY* __restrict__ y, int64_t y_row,
                    int64_t y_head, int tokens, int heads, int in, int out) {
  __shared__ float xs[HP_TOKENS][HP_IN];
  __shared__ float ms[HP_IN][HP_OUT + 1];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.y, t0 = blockIdx.z * HP_TOKENS, o0 = blockIdx.x * HP_OUT;
  const int tid = threadIdx.x;
  const TM* mh = m + (int64_t)h * m_head;
  float acc[HP_TOKENS];
#pragma unroll
  for (int u = 0; u < HP_TOKENS; ++u) acc[u] = 0.f;
  for (int i0 = 0; i0 < in; i0 += HP_IN) {
    __syncthreads();
    for (int e = tid; e < HP_TOKENS * HP_IN; e += HP_OUT) {
      const int u = e / HP_IN, i = e % HP_IN;
      xs[u][i] = (t0 + u < tokens && i0 + i < in) ? to_f32(x[(int64_t)(t0 + u) * x_row + (int64_t)h * x_head + i0 + i]) : 0.f;
    }
    if (m_in == 1) {             // the inner index is the contiguous one: neighbouring threads take neighbouring i
      for (int e = tid; e < HP_IN * HP_OUT; e += HP_OUT) {
        const int o = e / HP_IN, i = e % HP_IN;
        ms[i][o] = (o0 + o < out && i0 + i < in) ? to_f32(mh[(int64_t)(i0 + i) * m_in + (int64_t)(o0 + o) * m_out]) : 0.f;
      }
    } else {
      for (int e = tid; e < HP_IN * HP_OUT; e += HP_OUT) {
        const int i = e / HP_OUT, o = e % HP_OUT;
        ms[i][o] = (o0 + o < out && i0 + i < in) ? to_f32(mh[(int64_t)(i0 + i) * m_in + (int64_t)(o0 + o) * m_out]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll 8
    for (int i = 0; i < HP_IN; ++i) {
      const float w = ms[i][tid];
#pragma unroll
      for (int u = 0; u < HP_TOKENS; ++u) acc[u] = fmaf(xs[u][i], w, acc[u]);
    }
  }
  if (o0 + tid >= out) return;
#pragma unroll
  for (int u = 0; u < HP_TOKENS; ++u) {
    if (t0 + u >= tokens) break;
    const float g = gate != nullptr ? gate[(int64_t)(t0 + u) * heads + h] : 1.f;
    y[(int64_t)(t0 + u) * y_row + (int64_t)h * y_head + o0 + tid] = from_f32<TY>(acc[u] * g);
  }
}

__device__ __forceinline__ float dot_row(const float* __restrict__ q, const float* __restrict__ k, int d) {
  float s = 0.f;
  int i = 0;
  if (d % 4 == 0) {
    const float4* k4 = reinterpret_cast<const float4*>(k);
    for (; i < d; i += 4) {
      const float4 v = k4[i >> 2];
      s = fmaf(q[i], v.x, s);
      s = fmaf(q[i + 1], v.y, s);
      s = fmaf(q[i + 2], v.z, s);
      s = fmaf(q[i + 3], v.w, s);
    }
  }
  for (; i < d; ++i) s = fmaf(q[i], k[i], s);
  return s;
}
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const bf16* __restrict__ k, int d) {
  float s = 0.f;
  int i = 0;
  if (d % 8 == 0) {
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
    for (; i < d; i += 8) {
      const uint4 raw = k8[i >> 3];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        s = fmaf(q[i + 2 * j], f.x, s);
        s = fmaf(q[i + 2 * j + 1], f.y, s);
      }
    }
  }
  for (; i < d; ++i) s = fmaf(q[i], __bfloat162float(k[i]), s);
  return s;
}

// qk [rows, heads, rank + rot]: the query in latent form, then its rotated part. out float32
// [rows, heads, rank]: sum_j p_j c_j. RW = ceil(rank / 32) rounded up to the template's bucket.
template <typename T, int RW>
__global__ void __launch_bounds__(WARPS * 32)
latent_attend_kernel(const T* __restrict__ qk, const T* __restrict__ c_cache, const T* __restrict__ r_cache,
                     float* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ request_of,
                     const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                     const int* __restrict__ token_list, int tokens, int heads, int rank, int rot, float scale_log2,
                     int window, float* __restrict__ partial, int segment, unsigned* status) {
  extern __shared__ float q_smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
  if (wid >= (int64_t)tokens * heads) return;
  const int t = token_list != nullptr ? token_list[wid / heads] : (int)(wid / heads), h = (int)(wid % heads);
  const int kw = rank + rot;
  float* qs = q_smem + warp * kw;
  const T* qrow = qk + ((int64_t)t * heads + h) * kw;
  for (int i = lane; i < kw; i += 32) qs[i] = to_f32(qrow[i]);
  __syncwarp();

  const int b = request_of[t];
  const int pos = positions[t];
  int kstart = first_visible_key(pos, window);
  int kend = pos;                                   // inclusive
  if (partial != nullptr) {                         // this warp's segment of the keys (a multiple of 32)
    kstart = max(kstart, (int)blockIdx.y * segment);
    kend = min(kend, (int)(blockIdx.y + 1) * segment - 1);
  }
  const int* table = block_table + (int64_t)b * max_pages;
  float m = -INFINITY, l = 0.f;
  float acc[RW];
#pragma unroll
  for (int i = 0; i < RW; ++i) acc[i] = 0.f;

  for (int j0 = (kstart / 32) * 32; j0 <= kend; j0 += 32) {
    const int j = j0 + lane;
    bool valid = j >= kstart && j <= kend;
    int64_t slot = 0;
    float s = -INFINITY;
    if (valid) {
      const int slot_in_table = j / page_size;
      const int page = slot_in_table < max_pages ? table[slot_in_table] : -1;
      if (page < 0 || page >= num_pages) {
        raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
        valid = false;
      } else {
        slot = (int64_t)page * page_size + (j % page_size);
        s = (dot_row(qs, c_cache + slot * rank, rank) + dot_row(qs + rank, r_cache + slot * rot, rot)) * scale_log2;
      }
    }
    const float tile_max = warp_max(s);
    if (tile_max == -INFINITY) continue;
    const float m_new = fmaxf(m, tile_max);
    const float alpha = exp2f(m - m_new);
    const float p = valid ? exp2f(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < RW; ++i) acc[i] *= alpha;
    const int last = min(31, kend - j0);
    for (int kk = 0; kk <= last; kk += 4) {
      float pk[4];
      const T* crow[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        pk[u] = __shfl_sync(0xffffffffu, p, kk + u);
        crow[u] = c_cache + __shfl_sync(0xffffffffu, slot, kk + u) * rank;
      }
#pragma unroll
      for (int i = 0; i < RW; ++i) {
        const int idx = lane + 32 * i;
        if (idx < rank) {
          float x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) x[u] = to_f32(crow[u][idx]);
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[i] = fmaf(pk[u], x[u], acc[i]);
        }
      }
    }
    m = m_new;
  }
  if (partial != nullptr) {
    float* rec = partial + (wid * gridDim.y + blockIdx.y) * (int64_t)(rank + 2);
    if (lane == 0) {
      rec[0] = m;
      rec[1] = l;
    }
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      const int idx = lane + 32 * i;
      if (idx < rank) rec[2 + idx] = acc[i];
    }
    return;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float* orow = out + ((int64_t)t * heads + h) * rank;
#pragma unroll
  for (int i = 0; i < RW; ++i) {
    const int idx = lane + 32 * i;
    if (idx < rank) orow[idx] = acc[i] * inv;
  }
}

// A row's segments joined: the largest of the segments' maxima first (lanes over segments), then
// every segment's sums weighted by 2^(its maximum - the largest) and added in segment order, then
// the division. A warp takes MERGE_SLICE elements of a row (blockIdx.y says which), so that the loads
// of a segment do not wait for the segment before it; with few rows a warp takes 32, and the
// rows still fill the GPU.
template <int MERGE_SLICE>
__global__ void __launch_bounds__(WARPS * 32)
latent_merge_kernel(const float* __restrict__ partial, int segments, float* __restrict__ out,
                    const int* __restrict__ token_list, int tokens, int heads, int rank) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
  if (wid >= (int64_t)tokens * heads) return;
  const int t = token_list != nullptr ? token_list[wid / heads] : (int)(wid / heads), h = (int)(wid % heads);
  const float* row = partial + wid * segments * (int64_t)(rank + 2);
  float top = -INFINITY;
  for (int s = lane; s < segments; s += 32) top = fmaxf(top, row[(int64_t)s * (rank + 2)]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
  const int first = blockIdx.y * MERGE_SLICE;
  float l = 0.f;
  float acc[MERGE_SLICE / 32];
#pragma unroll
  for (int i = 0; i < MERGE_SLICE / 32; ++i) acc[i] = 0.f;
  if (top != -INFINITY) {
    // 32 segments at a time: lane j reads segment j's maximum and sum, so that the loop over the
    // segments' sums waits for no scalar; the sums are added in segment order
    for (int base = 0; base < segments; base += 32) {
      const int mine = base + lane;
      const float ms = mine < segments ? row[(int64_t)mine * (rank + 2)] : -INFINITY;
      const float ls = mine < segments ? row[(int64_t)mine * (rank + 2) + 1] : 0.f;     // every record has its sum of weights
      const float weight = ms == -INFINITY ? 0.f : exp2f(ms - top);     // a segment without a visible key left no sums
      if (weight != 0.f) l = fmaf(ls, weight, l);
      const int count = min(32, segments - base);
#pragma unroll 8
      for (int j = 0; j < count; ++j) {
        const float c = __shfl_sync(0xffffffffu, weight, j);
        const float* rec = row + (int64_t)(base + j) * (rank + 2);
#pragma unroll
        for (int i = 0; i < MERGE_SLICE / 32; ++i) {
          const int idx = first + lane + 32 * i;
          const float v = (c != 0.f && idx < rank) ? rec[2 + idx] : 0.f;
          acc[i] = fmaf(v, c, acc[i]);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float* orow = out + ((int64_t)t * heads + h) * rank;
#pragma unroll
  for (int i = 0; i < MERGE_SLICE / 32; ++i) {
    const int idx = first + lane + 32 * i;
    if (idx < rank) orow[idx] = acc[i] * inv;
  }
}

void launch_merge(int64_t blocks, cudaStream_t stream, const float* partial, int segments, float* out, const int* token_list,
                  int tokens, int heads, int rank) {
  if (blocks * ((rank + 127) / 128) >= 2 * 148)
    vosti_launch(latent_merge_kernel<128>, dim3((unsigned)blocks, (rank + 127) / 128), dim3(WARPS * 32), 0, stream, partial,
                 segments, out, token_list, tokens, heads, rank);
  else
    vosti_launch(latent_merge_kernel<32>, dim3((unsigned)blocks, (rank + 31) / 32), dim3(WARPS * 32), 0, stream, partial,
                 segments, out, token_list, tokens, heads, rank);
}

template <typename T, int RW>
void launch_attend(dim3 grid, size_t smem, cudaStream_t stream, const void* qk, const void* c_cache, const void* r_cache,
                   float* out, const int* positions, const int* request_of, const int* block_table, int max_pages,
                   int page_size, int num_pages, const int* token_list, int tokens, int heads, int rank, int rot,
                   float scale_log2, int window, float* partial, int segment, unsigned* status) {
  vosti_launch(latent_attend_kernel<T, RW>, grid, dim3(WARPS * 32), smem, stream, (const T*)qk, (const T*)c_cache,
               (const T*)r_cache, out, positions, request_of, block_table, max_pages, page_size, num_pages, token_list,
               tokens, heads, rank, rot, scale_log2, window, partial, segment, status);
}

}  // namespace

constexpr int LATENT_MAX_RANK = 1024;

// proj [tokens, heads * (dim + rot) + rank + rot + heads] = q | down | gate; qk [tokens, heads, rank + rot]
// (the last rot columns of every head are written); gate float32 [tokens, heads]; caches
// [pages, 1, page_size, rank | rot] or null (a run that reads another layer's cache).
VOSTI_API int vosti_latent_prep(const void* proj, void* qk, float* gate, void* c_cache, void* r_cache, const void* norm_w,
                                int norm_f32, float eps, const int* positions, const int* slot_mapping, int64_t num_slots,
                                int tokens, int heads, int dim, int rot, int rank, const float* freq, float magnitude,
                                int is_f32, unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && heads > 0 && dim > 0 && rank > 0 && rot >= 0 && rot % 2 == 0, "latent_prep: bad sizes");
  VOSTI_REQUIRE(rot == 0 || freq != nullptr, "latent_prep: a rotation needs frequencies");
  VOSTI_REQUIRE(c_cache == nullptr || (r_cache != nullptr && slot_mapping != nullptr && norm_w != nullptr), "latent_prep: a cache needs slots and the norm's weight");
  if (tokens == 0) return VOSTI_OK;
  const int64_t stride = (int64_t)heads * (dim + rot) + rank + rot + heads;
  const size_t smem = (size_t)(rot > 0 ? rot : 1) * sizeof(float);
  if (is_f32)
    vosti_launch(latent_prep_kernel<float>, dim3(tokens), dim3(256), smem, stream, (const float*)proj, stride, (float*)qk, gate,
                 (float*)c_cache, (float*)r_cache, norm_w, norm_f32, eps, positions, slot_mapping, num_slots, heads, dim, rot, rank,
                 freq, magnitude, status);
  else
    vosti_launch(latent_prep_kernel<bf16>, dim3(tokens), dim3(256), smem, stream, (const bf16*)proj, stride, (bf16*)qk, gate,
                 (bf16*)c_cache, (bf16*)r_cache, norm_w, norm_f32, eps, positions, slot_mapping, num_slots, heads, dim, rot, rank,
                 freq, magnitude, status);
  VOSTI_LAUNCH_CHECK();
}

// y[t, h, o] = gate[t, h] * sum_i x[t, h, i] * m[h * m_head + i * m_in + o * m_out]; strides in elements.
// Types: x and y float32 or bfloat16 (x_f32, y_f32), m float32 or bfloat16 (m_f32).
VOSTI_API int vosti_head_project(const void* x, int x_f32, int64_t x_row, int64_t x_head, const void* m, int m_f32,
                                 int64_t m_head, int64_t m_in, int64_t m_out, const float* gate, void* y, int y_f32,
                                 int64_t y_row, int64_t y_head, int tokens, int heads, int in, int out,
                                 cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && heads > 0 && heads <= 65535 && in > 0 && out > 0, "head_project: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int token_tiles = (tokens + HP_TOKENS - 1) / HP_TOKENS;
  VOSTI_REQUIRE(token_tiles <= 65535, "head_project: too many tokens for one launch");
  const dim3 grid((out + HP_OUT - 1) / HP_OUT, heads, token_tiles), block(HP_OUT);
#define VOSTI_HP(TX, TM, TY)                                                                                          \
  vosti_launch(head_project_kernel<TX, TM, TY>, grid, block, 0, stream, (const TX*)x, x_row, x_head, (const TM*)m, m_head, \
               m_in, m_out, gate, (TY*)y, y_row, y_head, tokens, heads, in, out)
  if (x_f32 && m_f32 && y_f32) VOSTI_HP(float, float, float);
  else if (x_f32 && !m_f32 && y_f32) VOSTI_HP(float, bf16, float);
  else if (x_f32 && !m_f32 && !y_f32) VOSTI_HP(float, bf16, bf16);
  else if (!x_f32 && !m_f32 && !y_f32) VOSTI_HP(bf16, bf16, bf16);
  else if (!x_f32 && !m_f32 && y_f32) VOSTI_HP(bf16, bf16, float);
  else if (x_f32 && m_f32 && !y_f32) VOSTI_HP(float, float, bf16);
  else {
    vosti_set_error("head_project: this mix of types is not built");
    return VOSTI_UNSUPPORTED;
  }
#undef VOSTI_HP
  VOSTI_LAUNCH_CHECK();
}

// qk [rows, heads, rank + rot]; caches [pages, 1, page_size, rank | rot]; out float32 [rows, heads, rank].
// `token_list` (or null: all) names the `tokens` rows to compute. With `segments` > 1 the keys
// are cut into pieces of `segment` keys (a multiple of 32) and `scratch` holds
// tokens * heads * segments * (rank + 2) floats.
VOSTI_API int vosti_latent_attend(const void* qk, const void* c_cache, const void* r_cache, float* out, const int* positions,
                                  const int* request_of, const int* block_table, int max_pages, int page_size,
                                  int num_pages, const int* token_list, int tokens, int heads, int rank, int rot,
                                  float scale, int window, float* scratch, int segment, int segments, int is_f32,
                                  unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && heads > 0 && rank > 0 && rank <= LATENT_MAX_RANK && rot >= 0,
                "latent_attend: bad sizes heads=%d rank=%d (at most %d) rot=%d", heads, rank, LATENT_MAX_RANK, rot);
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "latent_attend: bad cache geometry");
  VOSTI_REQUIRE(segments >= 1 && segments <= 65535 && (segments == 1 || (scratch != nullptr && segment > 0 && segment % 32 == 0)),
                "latent_attend: key segments need scratch and a length that is a multiple of 32");
  if (tokens == 0) return VOSTI_OK;
  const int64_t warps = (int64_t)tokens * heads;
  const int64_t blocks = (warps + WARPS - 1) / WARPS;
  VOSTI_REQUIRE(blocks <= 0x7fffffffLL, "latent_attend: too many (token, head) pairs");
  const size_t smem = (size_t)WARPS * (rank + rot) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    const int most = WARPS * (LATENT_MAX_RANK + 1024) * (int)sizeof(float);
#define VOSTI_LA_ATTR(RW)                                                                                          \
  cudaFuncSetAttribute(latent_attend_kernel<float, RW>, cudaFuncAttributeMaxDynamicSharedMemorySize, most); \
  cudaFuncSetAttribute(latent_attend_kernel<bf16, RW>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    VOSTI_LA_ATTR(4) VOSTI_LA_ATTR(8) VOSTI_LA_ATTR(16) VOSTI_LA_ATTR(32)
#undef VOSTI_LA_ATTR
    configured = true;
  }
  VOSTI_REQUIRE(rot <= 1024, "latent_attend: the rotated part has at most 1024 elements");
  float* partial = segments > 1 ? scratch : nullptr;
  const dim3 grid((unsigned)blocks, segments > 1 ? segments : 1);
  const int rw = rank <= 128 ? 4 : rank <= 256 ? 8 : rank <= 512 ? 16 : 32;
#define VOSTI_LA(RW)                                                                                                    \
  do {                                                                                                                  \
    if (is_f32)                                                                                                         \
      launch_attend<float, RW>(grid, smem, stream, qk, c_cache, r_cache, out, positions, request_of, block_table,       \
                               max_pages, page_size, num_pages, token_list, tokens, heads, rank, rot, scale * LOG2E,    \
                               window, partial, segment, status);                                                       \
    else                                                                                                                \
      launch_attend<bf16, RW>(grid, smem, stream, qk, c_cache, r_cache, out, positions, request_of, block_table,        \
                              max_pages, page_size, num_pages, token_list, tokens, heads, rank, rot, scale * LOG2E,     \
                              window, partial, segment, status);                                                        \
    if (segments > 1) {                                                                                                 \
      cudaError_t e = cudaGetLastError();                                                                               \
      if (e != cudaSuccess) { vosti_set_error("%s", cudaGetErrorString(e)); return (int)e; }                            \
      launch_merge(blocks, stream, partial, segments, out, token_list, tokens, heads, rank);                           \
    }                                                                                                                   \
  } while (0)
  if (rw == 4) VOSTI_LA(4);
  else if (rw == 8) VOSTI_LA(8);
  else if (rw == 16) VOSTI_LA(16);
  else VOSTI_LA(32);
#undef VOSTI_LA
  VOSTI_LAUNCH_CHECK();
}

// The merge alone, for a kernel that left the (m, l, sum) records itself: partial float32
// [tokens * heads, segments, rank + 2]; out float32 [tokens, heads, rank].
VOSTI_API int vosti_latent_merge(const float* partial, int segments, float* out, int tokens, int heads, int rank,
                                 cudaStream_t stream) {
  VOSTI_REQUIRE(partial != nullptr && segments >= 1 && tokens >= 0 && heads > 0 && rank > 0 && rank <= LATENT_MAX_RANK,
                "latent_merge: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int64_t blocks = ((int64_t)tokens * heads + WARPS - 1) / WARPS;
  VOSTI_REQUIRE(blocks <= 0x7fffffffLL, "latent_merge: too many (token, head) pairs");
  launch_merge(blocks, stream, partial, segments, out, nullptr, tokens, heads, rank);
  VOSTI_LAUNCH_CHECK();
}
