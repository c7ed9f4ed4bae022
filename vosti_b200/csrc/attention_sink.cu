// Paged causal attention with optional additions, and key and value heads of different widths:
//   * a rotation of the first 2 * rot_half elements of every query and key head, in pairs
//     (i, i + rot_half), by the angle position * freq[i] formed in float32 (no table, so no limit
//     on positions);
//   * a chunked mask instead of a window: a query sees the keys of its own chunk of positions
//     only (handed down as a negative window, see first_visible_key);
//   * a query temperature: the query at position p is multiplied by
//     1 + coef * ln(floor((p + 1) / every) + 1);
//   * a learned bias per (distance, head) added to the scaled score. The host hands a table
//     bias[head][min(distance, last)] (already in base-2 units): beyond `last` the bias no
//     longer changes, so the table is as long as the distances that differ;
//   * a sink: one more term exp(sink[head]) in the softmax denominator, with no key or value.
//
// Kernels: the projection's post-pass (temperature, keys and values into their cache slots)
// and the attention itself on the CUDA cores, one warp per (query token, query head), float32
// arithmetic for both storage types. A tile is 32 keys aligned to the absolute key index, so a
// row's order of arithmetic depends on its position only, not on how the prompt was cut or
// what else is in the batch. With few query rows (decoding) the keys are cut into segments of
// a fixed length, one warp per (token, head, segment), and a second kernel merges a row's
// segments in order; the sink joins at the merge. (Head sizes 64 and 128 in bfloat16 take the
// tensor-memory kernel of attention_prefill_tc.cu for their long rows instead.)
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_W = 256;          // widest key or value head
constexpr float LOG2E = 1.4426950408889634f;

// q . k for one key row; 16-byte loads when the row's width allows them.
__device__ __forceinline__ float dot_key(const float* __restrict__ q, const float* __restrict__ k, int d) {
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
__device__ __forceinline__ float dot_key(const float* __restrict__ q, const bf16* __restrict__ k, int d) {
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

template <typename T>
__global__ void __launch_bounds__(256)
qkv_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                 const int* __restrict__ positions, const int* __restrict__ slot_mapping, int64_t num_slots,
                 int page_size, int nq, int nkv, int dk, int dv, float temp_coef, int temp_every, unsigned* status,
                 const float* __restrict__ freq, int rot_half, float magnitude, const T* __restrict__ v_first,
                 int64_t v_first_stride, float v_mix) {
  extern __shared__ float turn[];            // [2 * rot_half]: cosines, then sines, of this token's angles
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int wq = nq * dk, wk = nkv * dk, wv = nkv * dv;
  const T* row = qkv + (int64_t)t * (wq + wk + wv);
  float temp = 1.f;
  if (temp_coef != 0.f) temp = 1.f + temp_coef * logf((float)((positions[t] + 1) / temp_every + 1));
  if (rot_half > 0) {
    const float p = (float)positions[t];
    for (int i = threadIdx.x; i < rot_half; i += blockDim.x) {
      const float angle = p * freq[i];
      turn[i] = cosf(angle) * magnitude;
      turn[rot_half + i] = sinf(angle) * magnitude;
    }
    __syncthreads();
  }
  // element i of a row of heads of width dk, turned if it lies in the rotated part of its head
  auto turned = [&](const T* src, int i) {
    const int j = i % dk;
    const float x = to_f32(src[i]);
    if (j < rot_half) return x * turn[j] - to_f32(src[i + rot_half]) * turn[rot_half + j];
    if (j < 2 * rot_half) return x * turn[j - rot_half] + to_f32(src[i - rot_half]) * turn[j];
    return x;
  };
  // bfloat16 rows whose widths allow it move as 16-byte words (8 elements)
  // (a rotated half must then be whole words too, so that a word's partner is a word)
  const bool vec = rot_half % 8 == 0 && sizeof(T) == 2 && dk % 8 == 0 && dv % 8 == 0;
  // word i (8 elements) of a row of heads of width dk, turned if it lies in the rotated part, times `by`
  auto turned_word = [&](const uint4* src, int i, float by) {
    uint4 raw = src[i];
    const int j = (i * 8) % dk;
    if (j >= 2 * rot_half && by == 1.f) return raw;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
    if (j < 2 * rot_half) {
      const bool low = j < rot_half;
      const uint4 other = src[low ? i + rot_half / 8 : i - rot_half / 8];
      const __nv_bfloat162* o = reinterpret_cast<const __nv_bfloat162*>(&other);
      const int a = low ? j : j - rot_half;                      // index of the angle of the word's first pair
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = __bfloat1622float2(p[e]), y = __bfloat1622float2(o[e]);
        const float c0 = turn[a + 2 * e], c1 = turn[a + 2 * e + 1], s0 = turn[rot_half + a + 2 * e], s1 = turn[rot_half + a + 2 * e + 1];
        const float r0 = low ? x.x * c0 - y.x * s0 : x.x * c0 + y.x * s0;
        const float r1 = low ? x.y * c1 - y.y * s1 : x.y * c1 + y.y * s1;
        p[e] = __floats2bfloat162_rn(r0 * by, r1 * by);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        p[e] = __floats2bfloat162_rn(f.x * by, f.y * by);
      }
    }
    return raw;
  };
  if (vec) {
    const uint4* src = reinterpret_cast<const uint4*>(row);
    uint4* dst = reinterpret_cast<uint4*>(q_out + (int64_t)t * wq);
    for (int i = threadIdx.x; i < wq / 8; i += blockDim.x) dst[i] = turned_word(src, i, temp);
  } else {
    for (int i = threadIdx.x; i < wq; i += blockDim.x) q_out[(int64_t)t * wq + i] = from_f32<T>(turned(row, i) * temp);
  }
  if (k_cache == nullptr) return;
  const int64_t slot = slot_mapping[t];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
    return;
  }
  const int64_t page = slot / page_size, offset = slot % page_size;
  if (vec) {
    const uint4* src = reinterpret_cast<const uint4*>(row);
    const int k8 = dk / 8, v8 = dv / 8;
    for (int i = threadIdx.x; i < wk / 8; i += blockDim.x) {
      const int g = i / k8, c = i % k8;
      reinterpret_cast<uint4*>(k_cache + ((page * nkv + g) * page_size + offset) * dk)[c] = turned_word(src + wq / 8, i, 1.f);
    }
    const bool mix_words = v_first != nullptr && v_first_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(v_first) & 15) == 0;
    for (int i = threadIdx.x; i < wv / 8; i += blockDim.x) {
      const int g = i / v8, c = i % v8;
      uint4 raw = src[(wq + wk) / 8 + i];
      if (mix_words) {
        const uint4 other = reinterpret_cast<const uint4*>(v_first + (int64_t)t * v_first_stride)[i];
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
        const __nv_bfloat162* o = reinterpret_cast<const __nv_bfloat162*>(&other);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __bfloat1622float2(p[e]), y = __bfloat1622float2(o[e]);
          p[e] = __floats2bfloat162_rn((1.f - v_mix) * x.x + v_mix * y.x, (1.f - v_mix) * x.y + v_mix * y.y);
        }
      } else if (v_first != nullptr) {
        bf16* p = reinterpret_cast<bf16*>(&raw);
        for (int e = 0; e < 8; ++e)
          p[e] = __float2bfloat16_rn((1.f - v_mix) * __bfloat162float(p[e]) +
                                     v_mix * to_f32(v_first[(int64_t)t * v_first_stride + i * 8 + e]));
      }
      reinterpret_cast<uint4*>(v_cache + ((page * nkv + g) * page_size + offset) * dv)[c] = raw;
    }
    return;
  }
  for (int i = threadIdx.x; i < wk; i += blockDim.x) {
    const int g = i / dk, c = i % dk;
    k_cache[((page * nkv + g) * page_size + offset) * dk + c] = rot_half > 0 ? from_f32<T>(turned(row + wq, i)) : row[wq + i];
  }
  for (int i = threadIdx.x; i < wv; i += blockDim.x) {
    const int g = i / dv, c = i % dv;
    T v = row[wq + wk + i];
    if (v_first != nullptr) v = from_f32<T>((1.f - v_mix) * to_f32(v) + v_mix * to_f32(v_first[(int64_t)t * v_first_stride + i]));
    v_cache[((page * nkv + g) * page_size + offset) * dv + c] = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_sink_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                      T* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ request_of,
                      const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                      const int* __restrict__ token_list, int tokens,
                      int nq, int nkv, int dk, int dv, float scale_log2, int window, const float* __restrict__ bias,
                      int bias_last, const float* __restrict__ sink, float* __restrict__ partial, int segment,
                      unsigned* status) {
  extern __shared__ float q_smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
  if (wid >= (int64_t)tokens * nq) return;
  const int t = token_list != nullptr ? token_list[wid / nq] : (int)(wid / nq), h = (int)(wid % nq);
  const int g = h / (nq / nkv);
  float* qs = q_smem + warp * dk;
  const T* qrow = q + ((int64_t)t * nq + h) * dk;
  for (int i = lane; i < dk; i += 32) qs[i] = to_f32(qrow[i]);
  __syncwarp();

  const int b = request_of[t];
  const int pos = positions[t];
  int kstart = first_visible_key(pos, window);
  int kend = pos;                                   // inclusive
  if (partial != nullptr) {                         // this warp's segment of the keys (segment: a multiple of 32)
    kstart = max(kstart, (int)blockIdx.y * segment);
    kend = min(kend, (int)(blockIdx.y + 1) * segment - 1);
  }
  const int* table = block_table + (int64_t)b * max_pages;
  const float* bias_h = bias != nullptr ? bias + (int64_t)h * (bias_last + 1) : nullptr;

  float m = -INFINITY, l = 0.f;
  float acc[MAX_W / 32];
#pragma unroll
  for (int i = 0; i < MAX_W / 32; ++i) acc[i] = 0.f;

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
        slot = ((int64_t)page * nkv + g) * page_size + (j % page_size);   // row of (page, head, offset)
        s = dot_key(qs, k_cache + slot * dk, dk) * scale_log2;
        if (bias_h != nullptr) s += bias_h[min(pos - j, bias_last)];
      }
    }
    const float tile_max = warp_max(s);
    if (tile_max == -INFINITY) continue;  // nothing visible here: state untouched
    const float m_new = fmaxf(m, tile_max);
    const float alpha = exp2f(m - m_new);
    const float p = valid ? exp2f(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_W / 32; ++i) acc[i] *= alpha;
    const int last = min(31, kend - j0);
    // four keys at a time, so that their value rows are in flight together (keys past the
    // end have p = 0 and slot 0, a row that exists)
    for (int kk = 0; kk <= last; kk += 4) {
      float pk[4];
      const T* vrow[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        pk[u] = __shfl_sync(0xffffffffu, p, kk + u);
        vrow[u] = v_cache + __shfl_sync(0xffffffffu, slot, kk + u) * dv;
      }
#pragma unroll
      for (int i = 0; i < MAX_W / 32; ++i) {
        const int idx = lane + 32 * i;
        if (idx < dv) {
          float x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) x[u] = to_f32(vrow[u][idx]);
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[i] = fmaf(pk[u], x[u], acc[i]);
        }
      }
    }
    m = m_new;
  }
  if (partial != nullptr) {
    // one record per (row, segment): maximum, sum, then the unnormalised values
    float* rec = partial + (wid * gridDim.y + blockIdx.y) * (int64_t)(dv + 2);
    if (lane == 0) {
      rec[0] = m;
      rec[1] = l;
    }
#pragma unroll
    for (int i = 0; i < MAX_W / 32; ++i) {
      const int idx = lane + 32 * i;
      if (idx < dv) rec[2 + idx] = acc[i];
    }
    return;
  }
  if (sink != nullptr) {
    // the sink has a logit and nothing else: it joins the denominator once
    const float s = sink[h] * LOG2E;
    const float m_new = fmaxf(m, s);
    const float alpha = exp2f(m - m_new);
    l = l * alpha + exp2f(s - m_new);
#pragma unroll
    for (int i = 0; i < MAX_W / 32; ++i) acc[i] *= alpha;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = out + ((int64_t)t * nq + h) * dv;
#pragma unroll
  for (int i = 0; i < MAX_W / 32; ++i) {
    const int idx = lane + 32 * i;
    if (idx < dv) orow[idx] = from_f32<T>(acc[i] * inv);
  }
}
// A row's segments in segment order, then the sink, then the division.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_sink_merge_kernel(const float* __restrict__ partial, int segments, T* __restrict__ out,
                            const int* __restrict__ token_list, int tokens, int nq, int dv,
                            const float* __restrict__ sink) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
  if (wid >= (int64_t)tokens * nq) return;
  const int t = token_list != nullptr ? token_list[wid / nq] : (int)(wid / nq), h = (int)(wid % nq);
  float m = -INFINITY, l = 0.f;
  float acc[MAX_W / 32];
#pragma unroll
  for (int i = 0; i < MAX_W / 32; ++i) acc[i] = 0.f;
  for (int s = 0; s < segments; ++s) {
    const float* rec = partial + (wid * segments + s) * (int64_t)(dv + 2);
    const float ms = rec[0], ls = rec[1];
    if (ms == -INFINITY) continue;
    const float m_new = fmaxf(m, ms);
    const float a = exp2f(m - m_new), c = exp2f(ms - m_new);
    l = l * a + ls * c;
#pragma unroll
    for (int i = 0; i < MAX_W / 32; ++i) {
      const int idx = lane + 32 * i;
      if (idx < dv) acc[i] = acc[i] * a + rec[2 + idx] * c;
    }
    m = m_new;
  }
  if (sink != nullptr) {
    const float s = sink[h] * LOG2E;
    const float m_new = fmaxf(m, s);
    const float a = exp2f(m - m_new);
    l = l * a + exp2f(s - m_new);
#pragma unroll
    for (int i = 0; i < MAX_W / 32; ++i) acc[i] *= a;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = out + ((int64_t)t * nq + h) * dv;
#pragma unroll
  for (int i = 0; i < MAX_W / 32; ++i) {
    const int idx = lane + 32 * i;
    if (idx < dv) orow[idx] = from_f32<T>(acc[i] * inv);
  }
}
}  // namespace

// qkv: [tokens, nq*dk + nkv*dk + nkv*dv]; q_out: [tokens, nq*dk]; caches [pages, nkv, page_size, dk | dv].
VOSTI_API int vosti_qkv_store(const void* qkv, void* q_out, void* k_cache, void* v_cache, const int* positions,
                              const int* slot_mapping, int64_t num_slots, int page_size, int tokens, int nq, int nkv,
                              int dk, int dv, float temp_coef, int temp_every, int is_f32, unsigned* status,
                              const float* freq, int rot_half, float magnitude, const void* v_first, int64_t v_first_stride,
                              float v_mix, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && nq > 0 && nkv >= 0 && dk > 0 && dv > 0, "qkv_store: bad sizes");
  VOSTI_REQUIRE(temp_coef == 0.f || (temp_every > 0 && positions != nullptr), "qkv_store: the temperature needs positions and a positive period");
  VOSTI_REQUIRE(k_cache == nullptr || (v_cache != nullptr && slot_mapping != nullptr && page_size > 0), "qkv_store: a cache needs slots");
  VOSTI_REQUIRE(rot_half >= 0 && 2 * rot_half <= dk && (rot_half == 0 || (freq != nullptr && positions != nullptr)),
                "qkv_store: the rotation takes at most the whole head and needs frequencies and positions");
  if (tokens == 0) return VOSTI_OK;
  const size_t turn_bytes = (size_t)2 * rot_half * sizeof(float);
  if (is_f32)
    vosti_launch(qkv_store_kernel<float>, dim3(tokens), dim3(256), turn_bytes, stream, (const float*)qkv, (float*)q_out, (float*)k_cache,
                 (float*)v_cache, positions, slot_mapping, num_slots, page_size, nq, nkv, dk, dv, temp_coef, temp_every, status, freq,
                 rot_half, magnitude, (const float*)v_first, v_first_stride, v_mix);
  else
    vosti_launch(qkv_store_kernel<bf16>, dim3(tokens), dim3(256), turn_bytes, stream, (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache,
                 (bf16*)v_cache, positions, slot_mapping, num_slots, page_size, nq, nkv, dk, dv, temp_coef, temp_every, status, freq,
                 rot_half, magnitude, (const bf16*)v_first, v_first_stride, v_mix);
  VOSTI_LAUNCH_CHECK();
}

// q: [rows, nq, dk]; out: [rows, nq, dv]; bias: float32 [nq, bias_last + 1] in natural-log units
// times log2(e), or null; sink: float32 [nq] in natural-log units, or null. `token_list` (or
// null: all of them) names the `tokens` rows to compute. With `segments` > 1 the keys are cut
// into pieces of `segment` keys (a multiple of 32) and `scratch` holds tokens * nq * segments *
// (dv + 2) floats.
VOSTI_API int vosti_attention_sink(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                                   const int* request_of, const int* block_table, int max_pages, int page_size,
                                   int num_pages, const int* token_list, int tokens, int nq, int nkv, int dk, int dv,
                                   float scale, int window, const float* bias, int bias_last, const float* sink,
                                   float* scratch, int segment, int segments, int is_f32, unsigned* status,
                                   cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention: bad head counts nq=%d nkv=%d", nq, nkv);
  VOSTI_REQUIRE(dk > 0 && dv > 0 && dk <= MAX_W && dv <= MAX_W, "attention: head widths %d / %d must be at most %d", dk, dv, MAX_W);
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention: bad cache geometry");
  VOSTI_REQUIRE(bias == nullptr || bias_last >= 0, "attention: bad bias table");       // (window < 0: a chunk)
  VOSTI_REQUIRE(segments >= 1 && segments <= 65535 && (segments == 1 || (scratch != nullptr && segment > 0 && segment % 32 == 0)),
                "attention: key segments need scratch and a length that is a multiple of 32");
  if (tokens == 0) return VOSTI_OK;
  const int64_t warps = (int64_t)tokens * nq;
  const int64_t blocks = (warps + WARPS - 1) / WARPS;
  VOSTI_REQUIRE(blocks <= 0x7fffffffLL, "attention: too many (token, head) pairs");
  const size_t smem = (size_t)WARPS * dk * sizeof(float);
  float* partial = segments > 1 ? scratch : nullptr;
  const dim3 grid((unsigned)blocks, segments > 1 ? segments : 1);
  if (is_f32)
    vosti_launch(attention_sink_kernel<float>, grid, dim3(WARPS * 32), smem, stream, (const float*)q,
                 (const float*)k_cache, (const float*)v_cache, (float*)out, positions, request_of, block_table, max_pages,
                 page_size, num_pages, token_list, tokens, nq, nkv, dk, dv, scale * LOG2E, window, bias, bias_last, sink,
                 partial, segment, status);
  else
    vosti_launch(attention_sink_kernel<bf16>, grid, dim3(WARPS * 32), smem, stream, (const bf16*)q,
                 (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, positions, request_of, block_table, max_pages,
                 page_size, num_pages, token_list, tokens, nq, nkv, dk, dv, scale * LOG2E, window, bias, bias_last, sink,
                 partial, segment, status);
  if (segments > 1) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { vosti_set_error("%s", cudaGetErrorString(e)); return (int)e; }
    if (is_f32)
      vosti_launch(attention_sink_merge_kernel<float>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
                   (const float*)partial, segments, (float*)out, token_list, tokens, nq, dv, sink);
    else
      vosti_launch(attention_sink_merge_kernel<bf16>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
                   (const float*)partial, segments, (bf16*)out, token_list, tokens, nq, dv, sink);
  }
  VOSTI_LAUNCH_CHECK();
}
