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
//   * a sink: one more term exp(sink[head]) in the softmax denominator, with no key or value;
//   * two score maps a head over the same values (differential attention), combined after the
//     softmax, and a finish of the head's output: unit root mean square, a sigmoid gate (HeadFinish);
//   * a projection post-pass by heads (qkv_heads): bias, per-head RMS norm with a shared weight,
//     rotation in pairs (i, i + n / 2) or (2i, 2i + 1), from a float32 product or its unsummed K splits.
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

__device__ __forceinline__ float4 load_four(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load_four(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store_four(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store_four(bf16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const unsigned*>(&lo);
  raw.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// What may follow a head's attention before the output projection, in float32:
//   * with two score maps a head (differential attention): o = a1 - lambda * a2, a1 and a2 the two
//     maps' softmax-weighted sums of the same values;
//   * `unit_norm`: o / sqrt(mean(o^2) + eps) over the head's values (no weight), times `out_scale`;
//   * `gate`: o * sigmoid(gate[t, h * dv + i]), the gate a product of the same input (float32 or
//     bfloat16 rows `gate_stride` elements apart).
struct HeadFinish {
  float lambda;
  float out_scale;
  float eps;
  int unit_norm;
  const void* gate;
  int gate_f32;
  long long gate_stride;
};

// acc[m][i]: map m's unnormalised sum for value element lane + 32 i; inv[m] = 1 / its denominator. One warp.
template <typename T, int MAPS>
__device__ __forceinline__ void finish_head(const float (&acc)[MAPS][MAX_W / 32], const float (&inv)[MAPS], const HeadFinish& f,
                                            int t, int h, int dv, T* __restrict__ orow) {
  const int lane = threadIdx.x & 31;
  float o[MAX_W / 32];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_W / 32; ++i) {
    o[i] = acc[0][i] * inv[0];
    if (MAPS == 2) o[i] -= f.lambda * (acc[MAPS - 1][i] * inv[MAPS - 1]);
    if (lane + 32 * i < dv) ss += o[i] * o[i];
  }
  float by = 1.f;
  if (f.unit_norm) by = f.out_scale / sqrtf(warp_sum(ss) / (float)dv + f.eps);
#pragma unroll
  for (int i = 0; i < MAX_W / 32; ++i) {
    const int idx = lane + 32 * i;
    if (idx < dv) {
      float y = f.unit_norm ? o[i] * by : o[i];
      if (f.gate != nullptr) y *= 1.f / (1.f + expf(-load_flex(f.gate, f.gate_f32, (int64_t)t * f.gate_stride + (int64_t)h * dv + idx)));
      orow[idx] = from_f32<T>(y);
    }
  }
}

// The same on attention outputs another kernel wrote: a [tokens, nq * MAPS, a_width] -> out [tokens, nq, dv],
// of a's rows the first dv elements. pair_group 0: head h's maps are rows h * MAPS + m; pair_group r > 0
// (maps that ran as heads of their own, grouped by kv head): rows h + (h / r) * r + m * r.
template <typename T, int MAPS>
__global__ void __launch_bounds__(WARPS * 32)
head_finish_kernel(const T* __restrict__ a, T* __restrict__ out, int tokens, int nq, int dv, int a_width, int pair_group,
                   HeadFinish f) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
  if (wid >= (int64_t)tokens * nq) return;
  const int t = (int)(wid / nq), h = (int)(wid % nq);
  if (dv % 4 == 0 && a_width % 4 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
      (f.gate == nullptr || (f.gate_f32 && f.gate_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(f.gate) & 15) == 0))) {
    // a lane takes four neighbouring elements (of every 128): whole words in and out
    constexpr int C = MAX_W / 128;
    float4 o[C];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const int i0 = 4 * lane + 128 * c;
      o[c] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i0 < dv) {
#pragma unroll
        for (int m = 0; m < MAPS; ++m) {
          const int64_t row = (int64_t)t * nq * MAPS + (pair_group > 0 ? h + (h / pair_group) * pair_group + m * pair_group : h * MAPS + m);
          const float4 v = load_four(a + row * a_width + i0);
          const float by = m == 0 ? 1.f : -f.lambda;
          o[c].x += by * v.x; o[c].y += by * v.y; o[c].z += by * v.z; o[c].w += by * v.w;
        }
        ss += (o[c].x * o[c].x + o[c].y * o[c].y) + (o[c].z * o[c].z + o[c].w * o[c].w);
      }
    }
    float by = 1.f;
    if (f.unit_norm) by = f.out_scale / sqrtf(warp_sum(ss) / (float)dv + f.eps);
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const int i0 = 4 * lane + 128 * c;
      if (i0 < dv) {
        float4 y = f.unit_norm ? make_float4(o[c].x * by, o[c].y * by, o[c].z * by, o[c].w * by) : o[c];
        if (f.gate != nullptr) {
          const float4 g = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(f.gate) + (int64_t)t * f.gate_stride + (int64_t)h * dv + i0);
          y.x *= 1.f / (1.f + expf(-g.x)); y.y *= 1.f / (1.f + expf(-g.y)); y.z *= 1.f / (1.f + expf(-g.z)); y.w *= 1.f / (1.f + expf(-g.w));
        }
        store_four(out + wid * dv + i0, y);
      }
    }
    return;
  }
  float acc[MAPS][MAX_W / 32], inv[MAPS];
#pragma unroll
  for (int m = 0; m < MAPS; ++m) {
    inv[m] = 1.f;
    const int64_t row = (int64_t)t * nq * MAPS + (pair_group > 0 ? h + (h / pair_group) * pair_group + m * pair_group : h * MAPS + m);
#pragma unroll
    for (int i = 0; i < MAX_W / 32; ++i) {
      const int idx = lane + 32 * i;
      acc[m][i] = idx < dv ? to_f32(a[row * a_width + idx]) : 0.f;
    }
  }
  finish_head<T, MAPS>(acc, inv, f, t, h, dv, out + wid * dv);
}

// After a q | k | v projection (float32 or the serving type, rows `proj_stride` elements apart so that
// further columns may follow), one block per token and a warp per head: add the projection's bias;
// RMS-norm every query and key head over its dk elements with a weight shared by all heads; turn the
// first 2 * rot_half elements of the head by position * freq[i], element i with i + rot_half or, with
// `interleaved`, 2i with 2i + 1 (cos and sin times `magnitude`); queries go to q_out
// [tokens, nq * maps * dk], keys and values to their cache slots. With `maps` score maps a head the
// projection holds nq * maps query heads and nkv * maps key heads, head by head, and the key cache's
// entry of a kv head is its maps keys side by side: [pages, nkv, page_size, maps * dk].
// `expanded`: every map is a head of its own for kernels that know one map a head and one width:
// queries go out dk_out wide (zeros after the first dk elements), the caches are
// [pages, nkv * maps, page_size, dk_out | dv_out], key head number kv * maps + m, a kv head's values
// written once for each of its maps, zeros after the first dk (dv) elements.
// R: elements of a head a lane holds (heads of up to 32 * R elements).
template <typename T, int R>
__global__ void __launch_bounds__(256, R <= 4 ? 4 : 2)
qkv_heads_kernel(const void* __restrict__ proj, int proj_f32, int64_t proj_stride, const float* __restrict__ bias,
                 T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ positions,
                 const int* __restrict__ slot_mapping, int64_t num_slots, int page_size, int nq, int nkv, int maps, int dk, int dv,
                 const void* __restrict__ q_norm, const void* __restrict__ k_norm, int norm_f32, float eps,
                 const float* __restrict__ freq, int rot_half, int interleaved, float magnitude, int expanded, int dk_out,
                 int dv_out, int splits, int64_t plane, float* __restrict__ extra_out, int extra_width, unsigned* status) {
  // splits > 1: proj is float32 [splits, tokens, proj_stride], the unsummed K splits of the product, added in
  // split order; the columns after q | k | v (extra_width of them: a gate) are then summed into extra_out.
  // The grid's y cuts a token's heads into pieces of one head a warp.
  extern __shared__ float heads_smem[];          // [2 * rot_half] cosines and sines, then [warps][dk] a head per warp
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* turn = heads_smem;
  float* buf = heads_smem + 2 * rot_half + warp * dk;
  if (rot_half > 0) {
    const float p = (float)positions[t];
    for (int i = threadIdx.x; i < rot_half; i += blockDim.x) {
      const float angle = p * freq[i];
      turn[i] = cosf(angle) * magnitude;
      turn[rot_half + i] = sinf(angle) * magnitude;
    }
    __syncthreads();
  }
  int64_t page = 0, offset = 0;
  bool store = k_cache != nullptr;
  if (store) {
    const int64_t slot = slot_mapping[t];
    if (slot < 0 || slot >= num_slots) {
      if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
      store = false;
    }
    page = slot / page_size;
    offset = slot % page_size;
  }
  const int nqm = nq * maps, nkm = nkv * maps;
  const int64_t wq = (int64_t)nqm * dk, wk = (int64_t)nkm * dk;
  // 16-byte words when everything is float32 and lies on 16-byte borders
  const bool vec4 = proj_f32 && (norm_f32 || (q_norm == nullptr && k_norm == nullptr)) && proj_stride % 4 == 0 && dk % 4 == 0 && dv % 4 == 0 &&
                    (rot_half == 0 || (interleaved ? rot_half % 2 == 0 : rot_half % 4 == 0)) && (!expanded || (dk_out % 4 == 0 && dv_out % 4 == 0)) &&
                    (reinterpret_cast<uintptr_t>(proj) & 15) == 0 && (bias == nullptr || (reinterpret_cast<uintptr_t>(bias) & 15) == 0) &&
                    (q_norm == nullptr || (reinterpret_cast<uintptr_t>(q_norm) & 15) == 0) && (k_norm == nullptr || (reinterpret_cast<uintptr_t>(k_norm) & 15) == 0);
  const int64_t row = (int64_t)t * proj_stride;
  const int pieces = extra_out != nullptr ? (extra_width + 32 * R - 1) / (32 * R) : 0;       // the extra columns, 32 * R a warp
  for (int hd = blockIdx.y * nwarps + warp; hd < nqm + nkm + nkv + pieces; hd += gridDim.y * nwarps) {
    if (hd >= nqm + nkm + nkv) {
      const int64_t off = wq + wk + (int64_t)nkv * dv;
      const int c0 = (hd - nqm - nkm - nkv) * 32 * R;
      float g[R];
#pragma unroll
      for (int j = 0; j < R; ++j) g[j] = c0 + lane + 32 * j < extra_width ? load_flex(proj, proj_f32, row + off + c0 + lane + 32 * j) : 0.f;
      for (int sp = 1; sp < splits; ++sp) {
        const float* p = reinterpret_cast<const float*>(proj) + sp * plane + row + off + c0;
#pragma unroll
        for (int j = 0; j < R; ++j)
          if (c0 + lane + 32 * j < extra_width) g[j] += p[lane + 32 * j];
      }
#pragma unroll
      for (int j = 0; j < R; ++j)
        if (c0 + lane + 32 * j < extra_width) extra_out[(int64_t)t * extra_width + c0 + lane + 32 * j] = g[j];
      continue;
    }
    if (hd >= nqm + nkm) {                         // a value head: bias, then its cache slot
      if (!store) continue;
      const int g = hd - nqm - nkm;
      const int64_t off = wq + wk + (int64_t)g * dv;
      if (vec4) {
        const float* pf = reinterpret_cast<const float*>(proj) + row + off;
        const int wide = expanded ? dv_out : dv;
        for (int i0 = 4 * lane; i0 < wide; i0 += 128) {
          float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i0 < dv) {
            x = *reinterpret_cast<const float4*>(pf + i0);
            for (int sp = 1; sp < splits; ++sp) {
              const float4 y = *reinterpret_cast<const float4*>(pf + sp * plane + i0);
              x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
            }
            if (bias != nullptr) {
              const float4 y = *reinterpret_cast<const float4*>(bias + off + i0);
              x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
            }
          }
          if (expanded) {
            for (int c = 0; c < maps; ++c) store_four(v_cache + ((page * nkm + g * maps + c) * page_size + offset) * dv_out + i0, x);
          } else {
            store_four(v_cache + ((page * nkv + g) * page_size + offset) * dv + i0, x);
          }
        }
        continue;
      }
      if (expanded) {
        for (int i = lane; i < dv_out; i += 32) {
          float x = 0.f;
          if (i < dv) {
            x = load_flex(proj, proj_f32, row + off + i);
            for (int sp = 1; sp < splits; ++sp) x += reinterpret_cast<const float*>(proj)[sp * plane + row + off + i];
            if (bias != nullptr) x += bias[off + i];
          }
          for (int c = 0; c < maps; ++c) v_cache[((page * nkm + g * maps + c) * page_size + offset) * dv_out + i] = from_f32<T>(x);
        }
        continue;
      }
      T* dst = v_cache + ((page * nkv + g) * page_size + offset) * dv;
      for (int i = lane; i < dv; i += 32) {
        float x = load_flex(proj, proj_f32, row + off + i);
        for (int sp = 1; sp < splits; ++sp) x += reinterpret_cast<const float*>(proj)[sp * plane + row + off + i];
        if (bias != nullptr) x += bias[off + i];
        dst[i] = from_f32<T>(x);
      }
      continue;
    }
    const bool is_q = hd < nqm;
    if (!is_q && !store) continue;
    const int64_t off = (int64_t)hd * dk;          // query heads, then key heads, in the projection's order
    const void* norm_w = is_q ? q_norm : k_norm;
    T* dst;
    if (is_q) {
      dst = expanded ? q_out + ((int64_t)t * nqm + hd) * dk_out : q_out + (int64_t)t * wq + off;
    } else {
      const int kh = hd - nqm, g = kh / maps, m = kh % maps;
      dst = expanded ? k_cache + ((page * nkm + kh) * page_size + offset) * dk_out
                     : k_cache + (((page * nkv + g) * page_size + offset) * maps + m) * dk;
    }
    if (expanded)
      for (int i = dk + lane; i < dk_out; i += 32) dst[i] = from_f32<T>(0.f);
    if (vec4) {
      // a lane takes four neighbouring elements (of every 128): 16-byte loads, one store of four
      constexpr int C = R / 4;
      const float* pf = reinterpret_cast<const float*>(proj) + row + off;
      float4 xv[C], nv[C];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const int i0 = 4 * lane + 128 * c;
        xv[c] = i0 < dk ? *reinterpret_cast<const float4*>(pf + i0) : make_float4(0.f, 0.f, 0.f, 0.f);
        nv[c] = (norm_w != nullptr && i0 < dk) ? *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(norm_w) + i0)
                                               : make_float4(1.f, 1.f, 1.f, 1.f);
      }
      for (int sp = 1; sp < splits; ++sp) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int i0 = 4 * lane + 128 * c;
          if (i0 < dk) {
            const float4 y = *reinterpret_cast<const float4*>(pf + sp * plane + i0);
            xv[c].x += y.x; xv[c].y += y.y; xv[c].z += y.z; xv[c].w += y.w;
          }
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const int i0 = 4 * lane + 128 * c;
        if (bias != nullptr && i0 < dk) {
          const float4 y = *reinterpret_cast<const float4*>(bias + off + i0);
          xv[c].x += y.x; xv[c].y += y.y; xv[c].z += y.z; xv[c].w += y.w;
        }
        ss += (xv[c].x * xv[c].x + xv[c].y * xv[c].y) + (xv[c].z * xv[c].z + xv[c].w * xv[c].w);
      }
      if (norm_w != nullptr) {
        const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dk + eps);
#pragma unroll
        for (int c = 0; c < C; ++c)
          xv[c] = make_float4(xv[c].x * inv * nv[c].x, xv[c].y * inv * nv[c].y, xv[c].z * inv * nv[c].z, xv[c].w * inv * nv[c].w);
      }
      if (rot_half > 0 && interleaved) {
        // both elements of a pair lie in the lane's four
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int i0 = 4 * lane + 128 * c;
          if (i0 < 2 * rot_half) {
            const float c0 = turn[i0 >> 1], c1 = turn[(i0 >> 1) + 1], s0 = turn[rot_half + (i0 >> 1)], s1 = turn[rot_half + (i0 >> 1) + 1];
            const float4 v = xv[c];
            xv[c] = make_float4(v.x * c0 - v.y * s0, v.y * c0 + v.x * s0, v.z * c1 - v.w * s1, v.w * c1 + v.z * s1);
          }
        }
      } else if (rot_half > 0) {
#pragma unroll
        for (int c = 0; c < C; ++c)
          if (4 * lane + 128 * c < dk) *reinterpret_cast<float4*>(buf + 4 * lane + 128 * c) = xv[c];
        __syncwarp();
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int i0 = 4 * lane + 128 * c;
          if (i0 < 2 * rot_half) {
            const bool first = i0 < rot_half;
            const int pair = first ? i0 : i0 - rot_half;
            const float4 o = *reinterpret_cast<const float4*>(buf + (first ? i0 + rot_half : i0 - rot_half));
            const float4 cs = *reinterpret_cast<const float4*>(turn + pair), sn = *reinterpret_cast<const float4*>(turn + rot_half + pair);
            const float4 v = xv[c];
            xv[c] = first ? make_float4(v.x * cs.x - o.x * sn.x, v.y * cs.y - o.y * sn.y, v.z * cs.z - o.z * sn.z, v.w * cs.w - o.w * sn.w)
                          : make_float4(v.x * cs.x + o.x * sn.x, v.y * cs.y + o.y * sn.y, v.z * cs.z + o.z * sn.z, v.w * cs.w + o.w * sn.w);
          }
        }
        __syncwarp();
      }
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const int i0 = 4 * lane + 128 * c;
        if (i0 < dk) store_four(dst + i0, xv[c]);
      }
      continue;
    }
    float x[R], nw[R];
    float ss = 0.f;
    // the loads of one split (and the norm's weights) are in flight together; splits are added in split order
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int i = lane + 32 * j;
      x[j] = i < dk ? load_flex(proj, proj_f32, row + off + i) : 0.f;
      nw[j] = (norm_w != nullptr && i < dk) ? load_flex(norm_w, norm_f32, i) : 1.f;
    }
    for (int sp = 1; sp < splits; ++sp) {
      const float* p = reinterpret_cast<const float*>(proj) + sp * plane + row + off;
#pragma unroll
      for (int j = 0; j < R; ++j)
        if (lane + 32 * j < dk) x[j] += p[lane + 32 * j];
    }
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int i = lane + 32 * j;
      if (i < dk) {
        if (bias != nullptr) x[j] += bias[off + i];
        ss += x[j] * x[j];
      }
    }
    if (norm_w != nullptr) {
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dk + eps);
#pragma unroll
      for (int j = 0; j < R; ++j) x[j] = x[j] * inv * nw[j];
    }
    if (rot_half > 0) {
#pragma unroll
      for (int j = 0; j < R; ++j)
        if (lane + 32 * j < dk) buf[lane + 32 * j] = x[j];
      __syncwarp();
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const int i = lane + 32 * j;
        if (i < 2 * rot_half) {
          const bool first = interleaved ? (i & 1) == 0 : i < rot_half;
          const int pair = interleaved ? i >> 1 : (first ? i : i - rot_half);
          const float other = buf[interleaved ? i ^ 1 : (first ? i + rot_half : i - rot_half)];
          const float c = turn[pair], sn = turn[rot_half + pair];
          x[j] = first ? x[j] * c - other * sn : x[j] * c + other * sn;
        }
      }
      __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int i = lane + 32 * j;
      if (i < dk) dst[i] = from_f32<T>(x[j]);
    }
  }
}

template <typename T, int MAPS>
__global__ void __launch_bounds__(WARPS * 32)
attention_sink_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                      T* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ request_of,
                      const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                      const int* __restrict__ token_list, int tokens,
                      int nq, int nkv, int dk, int dv, float scale_log2, int window, const float* __restrict__ bias,
                      int bias_last, const float* __restrict__ sink, float* __restrict__ partial, int segment,
                      unsigned* status, HeadFinish finish) {
  // MAPS score maps a head: the query row holds MAPS queries, a key entry MAPS keys side by side,
  // every map has a softmax of its own over the same values (a value row is loaded once for all).
  extern __shared__ float q_smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
  if (wid >= (int64_t)tokens * nq) return;
  const int t = token_list != nullptr ? token_list[wid / nq] : (int)(wid / nq), h = (int)(wid % nq);
  const int g = h / (nq / nkv);
  float* qs = q_smem + warp * MAPS * dk;
  const T* qrow = q + ((int64_t)t * nq + h) * MAPS * dk;
  for (int i = lane; i < MAPS * dk; i += 32) qs[i] = to_f32(qrow[i]);
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

  float m[MAPS], l[MAPS];
  float acc[MAPS][MAX_W / 32];
#pragma unroll
  for (int a = 0; a < MAPS; ++a) {
    m[a] = -INFINITY;
    l[a] = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_W / 32; ++i) acc[a][i] = 0.f;
  }

  for (int j0 = (kstart / 32) * 32; j0 <= kend; j0 += 32) {
    const int j = j0 + lane;
    bool valid = j >= kstart && j <= kend;
    int64_t slot = 0;
    float s[MAPS];
#pragma unroll
    for (int a = 0; a < MAPS; ++a) s[a] = -INFINITY;
    if (valid) {
      const int slot_in_table = j / page_size;
      const int page = slot_in_table < max_pages ? table[slot_in_table] : -1;
      if (page < 0 || page >= num_pages) {
        raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
        valid = false;
      } else {
        slot = ((int64_t)page * nkv + g) * page_size + (j % page_size);   // row of (page, head, offset)
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
          s[a] = dot_key(qs + a * dk, k_cache + (slot * MAPS + a) * dk, dk) * scale_log2;
          if (bias_h != nullptr) s[a] += bias_h[min(pos - j, bias_last)];
        }
      }
    }
    float p[MAPS];
    bool any = false;
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
      const float tile_max = warp_max(s[a]);
      p[a] = 0.f;
      if (tile_max == -INFINITY) continue;  // nothing visible here: state untouched
      any = true;
      const float m_new = fmaxf(m[a], tile_max);
      const float alpha = exp2f(m[a] - m_new);
      p[a] = valid ? exp2f(s[a] - m_new) : 0.f;
      l[a] = l[a] * alpha + warp_sum(p[a]);
#pragma unroll
      for (int i = 0; i < MAX_W / 32; ++i) acc[a][i] *= alpha;
      m[a] = m_new;
    }
    if (!any) continue;
    const int last = min(31, kend - j0);
    // four keys at a time, so that their value rows are in flight together (keys past the
    // end have p = 0 and slot 0, a row that exists)
    for (int kk = 0; kk <= last; kk += 4) {
      float pk[MAPS][4];
      const T* vrow[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int a = 0; a < MAPS; ++a) pk[a][u] = __shfl_sync(0xffffffffu, p[a], kk + u);
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
          for (int a = 0; a < MAPS; ++a)
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[a][i] = fmaf(pk[a][u], x[u], acc[a][i]);
        }
      }
    }
  }
  if (partial != nullptr) {
    // one record per (row, segment, map): maximum, sum, then the unnormalised values
    float* rec = partial + (wid * gridDim.y + blockIdx.y) * (int64_t)(MAPS * (dv + 2));
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
      float* r = rec + a * (dv + 2);
      if (lane == 0) {
        r[0] = m[a];
        r[1] = l[a];
      }
#pragma unroll
      for (int i = 0; i < MAX_W / 32; ++i) {
        const int idx = lane + 32 * i;
        if (idx < dv) r[2 + idx] = acc[a][i];
      }
    }
    return;
  }
  float inv[MAPS];
#pragma unroll
  for (int a = 0; a < MAPS; ++a) {
    if (sink != nullptr) {
      // the sink has a logit and nothing else: it joins the denominator once
      const float sl = sink[h] * LOG2E;
      const float m_new = fmaxf(m[a], sl);
      const float alpha = exp2f(m[a] - m_new);
      l[a] = l[a] * alpha + exp2f(sl - m_new);
#pragma unroll
      for (int i = 0; i < MAX_W / 32; ++i) acc[a][i] *= alpha;
    }
    inv[a] = l[a] > 0.f ? 1.f / l[a] : 0.f;
  }
  finish_head<T, MAPS>(acc, inv, finish, t, h, dv, out + ((int64_t)t * nq + h) * dv);
}
// A row's segments in segment order, then the sink, then the division.
template <typename T, int MAPS>
__global__ void __launch_bounds__(WARPS * 32)
attention_sink_merge_kernel(const float* __restrict__ partial, int segments, T* __restrict__ out,
                            const int* __restrict__ token_list, int tokens, int nq, int dv,
                            const float* __restrict__ sink, HeadFinish finish) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
  if (wid >= (int64_t)tokens * nq) return;
  const int t = token_list != nullptr ? token_list[wid / nq] : (int)(wid / nq), h = (int)(wid % nq);
  float acc[MAPS][MAX_W / 32], inv[MAPS];
#pragma unroll
  for (int a = 0; a < MAPS; ++a) {
    float m = -INFINITY, l = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_W / 32; ++i) acc[a][i] = 0.f;
    for (int s = 0; s < segments; ++s) {
      const float* rec = partial + ((wid * segments + s) * MAPS + a) * (int64_t)(dv + 2);
      const float ms = rec[0], ls = rec[1];
      if (ms == -INFINITY) continue;
      const float m_new = fmaxf(m, ms);
      const float x = exp2f(m - m_new), c = exp2f(ms - m_new);
      l = l * x + ls * c;
#pragma unroll
      for (int i = 0; i < MAX_W / 32; ++i) {
        const int idx = lane + 32 * i;
        if (idx < dv) acc[a][i] = acc[a][i] * x + rec[2 + idx] * c;
      }
      m = m_new;
    }
    if (sink != nullptr) {
      const float s = sink[h] * LOG2E;
      const float m_new = fmaxf(m, s);
      const float x = exp2f(m - m_new);
      l = l * x + exp2f(s - m_new);
#pragma unroll
      for (int i = 0; i < MAX_W / 32; ++i) acc[a][i] *= x;
    }
    inv[a] = l > 0.f ? 1.f / l : 0.f;
  }
  finish_head<T, MAPS>(acc, inv, finish, t, h, dv, out + ((int64_t)t * nq + h) * dv);
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

static const HeadFinish NO_FINISH = {0.f, 1.f, 0.f, 0, nullptr, 0, 0};

template <typename T, int MAPS>
static cudaError_t attention_sink_launch(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                                         const int* request_of, const int* block_table, int max_pages, int page_size, int num_pages,
                                         const int* token_list, int tokens, int nq, int nkv, int dk, int dv, float scale, int window,
                                         const float* bias, int bias_last, const float* sink, float* partial, int segment,
                                         int segments, unsigned* status, const HeadFinish& finish, cudaStream_t stream) {
  const int64_t blocks = ((int64_t)tokens * nq + WARPS - 1) / WARPS;
  const size_t smem = (size_t)WARPS * MAPS * dk * sizeof(float);
  const dim3 grid((unsigned)blocks, segments > 1 ? segments : 1);
  vosti_launch(attention_sink_kernel<T, MAPS>, grid, dim3(WARPS * 32), smem, stream, (const T*)q, (const T*)k_cache, (const T*)v_cache,
               (T*)out, positions, request_of, block_table, max_pages, page_size, num_pages, token_list, tokens, nq, nkv, dk, dv,
               scale * LOG2E, window, bias, bias_last, sink, partial, segment, status, finish);
  if (segments > 1) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    vosti_launch(attention_sink_merge_kernel<T, MAPS>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, (const float*)partial,
                 segments, (T*)out, token_list, tokens, nq, dv, sink, finish);
  }
  return cudaGetLastError();
}

// q: [rows, nq, maps, dk]; caches [pages, nkv, page_size, maps * dk | dv]; out: [rows, nq, dv]; bias: float32
// [nq, bias_last + 1] in natural-log units
// times log2(e), or null; sink: float32 [nq] in natural-log units, or null. `token_list` (or
// null: all of them) names the `tokens` rows to compute. With `segments` > 1 the keys are cut
// into pieces of `segment` keys (a multiple of 32) and `scratch` holds tokens * nq * segments * maps *
// (dv + 2) floats. maps is 1 or 2 (see HeadFinish for what follows the softmax: lambda, the unit norm
// with eps and out_scale, the gate).
VOSTI_API int vosti_attention_maps(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                                   const int* request_of, const int* block_table, int max_pages, int page_size,
                                   int num_pages, const int* token_list, int tokens, int nq, int nkv, int maps, int dk, int dv,
                                   float scale, int window, const float* bias, int bias_last, const float* sink,
                                   float* scratch, int segment, int segments, float lambda, int unit_norm, float eps,
                                   float out_scale, const void* gate, int gate_f32, long long gate_stride, int is_f32,
                                   unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention: bad head counts nq=%d nkv=%d", nq, nkv);
  VOSTI_REQUIRE(maps == 1 || maps == 2, "attention: one or two score maps a head, not %d", maps);
  VOSTI_REQUIRE(dk > 0 && dv > 0 && dk <= MAX_W && dv <= MAX_W, "attention: head widths %d / %d must be at most %d", dk, dv, MAX_W);
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention: bad cache geometry");
  VOSTI_REQUIRE(bias == nullptr || bias_last >= 0, "attention: bad bias table");       // (window < 0: a chunk)
  VOSTI_REQUIRE(segments >= 1 && segments <= 65535 && (segments == 1 || (scratch != nullptr && segment > 0 && segment % 32 == 0)),
                "attention: key segments need scratch and a length that is a multiple of 32");
  VOSTI_REQUIRE(gate == nullptr || gate_stride >= (long long)nq * dv, "attention: the gate's rows are narrower than the heads");
  if (tokens == 0) return VOSTI_OK;
  VOSTI_REQUIRE(((int64_t)tokens * nq + WARPS - 1) / WARPS <= 0x7fffffffLL, "attention: too many (token, head) pairs");
  const HeadFinish finish = {lambda, out_scale, eps, unit_norm, gate, gate_f32, gate_stride};
  float* partial = segments > 1 ? scratch : nullptr;
  cudaError_t e;
#define VOSTI_SINK_ARGS q, k_cache, v_cache, out, positions, request_of, block_table, max_pages, page_size, num_pages, token_list, \
                        tokens, nq, nkv, dk, dv, scale, window, bias, bias_last, sink, partial, segment, segments, status, finish, stream
  if (is_f32) e = maps == 2 ? attention_sink_launch<float, 2>(VOSTI_SINK_ARGS) : attention_sink_launch<float, 1>(VOSTI_SINK_ARGS);
  else e = maps == 2 ? attention_sink_launch<bf16, 2>(VOSTI_SINK_ARGS) : attention_sink_launch<bf16, 1>(VOSTI_SINK_ARGS);
#undef VOSTI_SINK_ARGS
  if (e != cudaSuccess) { vosti_set_error("%s", cudaGetErrorString(e)); return (int)e; }
  return VOSTI_OK;
}

VOSTI_API int vosti_attention_sink(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                                   const int* request_of, const int* block_table, int max_pages, int page_size,
                                   int num_pages, const int* token_list, int tokens, int nq, int nkv, int dk, int dv,
                                   float scale, int window, const float* bias, int bias_last, const float* sink,
                                   float* scratch, int segment, int segments, int is_f32, unsigned* status,
                                   cudaStream_t stream) {
  return vosti_attention_maps(q, k_cache, v_cache, out, positions, request_of, block_table, max_pages, page_size, num_pages, token_list,
                              tokens, nq, nkv, 1, dk, dv, scale, window, bias, bias_last, sink, scratch, segment, segments,
                              NO_FINISH.lambda, 0, 0.f, 1.f, nullptr, 0, 0, is_f32, status, stream);
}

// a: [tokens, nq, maps, dv] attention outputs -> out [tokens, nq, dv] (see HeadFinish).
VOSTI_API int vosti_head_finish(const void* a, void* out, int tokens, int nq, int maps, int dv, int a_width, int pair_group,
                                float lambda, int unit_norm, float eps,
                                float out_scale, const void* gate, int gate_f32, long long gate_stride, int is_f32,
                                cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && nq > 0 && dv > 0 && dv <= MAX_W && (maps == 1 || maps == 2), "head_finish: bad sizes");
  VOSTI_REQUIRE(a_width >= dv && pair_group >= 0 && (pair_group == 0 || nq % pair_group == 0), "head_finish: bad input layout");
  VOSTI_REQUIRE(gate == nullptr || gate_stride >= (long long)nq * dv, "head_finish: the gate's rows are narrower than the heads");
  if (tokens == 0) return VOSTI_OK;
  const HeadFinish f = {lambda, out_scale, eps, unit_norm, gate, gate_f32, gate_stride};
  const unsigned blocks = (unsigned)(((int64_t)tokens * nq + WARPS - 1) / WARPS);
  if (is_f32) {
    if (maps == 2) vosti_launch(head_finish_kernel<float, 2>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const float*)a, (float*)out, tokens, nq, dv, a_width, pair_group, f);
    else vosti_launch(head_finish_kernel<float, 1>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const float*)a, (float*)out, tokens, nq, dv, a_width, pair_group, f);
  } else {
    if (maps == 2) vosti_launch(head_finish_kernel<bf16, 2>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const bf16*)a, (bf16*)out, tokens, nq, dv, a_width, pair_group, f);
    else vosti_launch(head_finish_kernel<bf16, 1>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const bf16*)a, (bf16*)out, tokens, nq, dv, a_width, pair_group, f);
  }
  VOSTI_LAUNCH_CHECK();
}

// proj: [tokens, >= (nq * maps + nkv * maps) * dk + nkv * dv] float32 or bfloat16, rows proj_stride elements apart; bias float32
// over the q | k | v columns, or null; q_norm / k_norm [dk] (float32 or bfloat16, both of one type), or null;
// freq float32 [rot_half], or rot_half 0. Outputs in the serving type: q_out [tokens, nq * maps * dk];
// caches [pages, nkv, page_size, maps * dk | dv] (null: queries only). `expanded` (see the kernel): q_out
// [tokens, nq * maps * dk_out], caches [pages, nkv * maps, page_size, dk_out | dv_out].
VOSTI_API int vosti_qkv_heads(const void* proj, int proj_f32, long long proj_stride, const float* bias, void* q_out, void* k_cache,
                              void* v_cache, const int* positions, const int* slot_mapping, int64_t num_slots, int page_size,
                              int tokens, int nq, int nkv, int maps, int dk, int dv, const void* q_norm, const void* k_norm,
                              int norm_f32, float eps, const float* freq, int rot_half, int interleaved, float magnitude,
                              int expanded, int dk_out, int dv_out, int splits, float* extra_out, int extra_width, int is_f32,
                              unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(!expanded || (dk_out >= dk && dv_out >= dv), "qkv_heads: expanded heads are at least as wide as the heads");
  VOSTI_REQUIRE(splits >= 1 && (splits == 1 || proj_f32), "qkv_heads: unsummed splits are float32");
  VOSTI_REQUIRE(extra_out == nullptr || (extra_width > 0 && proj_stride >= (long long)(nq + nkv) * maps * dk + (long long)nkv * dv + extra_width),
                "qkv_heads: the extra columns lie after q | k | v inside the projection's rows");
  const int64_t plane = (int64_t)tokens * proj_stride;
  VOSTI_REQUIRE(tokens >= 0 && nq > 0 && nkv >= 0 && maps >= 1 && dk > 0 && dv > 0 && dk <= MAX_W && dv <= MAX_W, "qkv_heads: bad sizes");
  VOSTI_REQUIRE(proj_stride >= (long long)(nq + nkv) * maps * dk + (long long)nkv * dv, "qkv_heads: the projection's rows are too narrow");
  VOSTI_REQUIRE(k_cache == nullptr || (v_cache != nullptr && slot_mapping != nullptr && page_size > 0), "qkv_heads: a cache needs slots");
  VOSTI_REQUIRE(rot_half >= 0 && 2 * rot_half <= dk && (rot_half == 0 || (freq != nullptr && positions != nullptr)),
                "qkv_heads: the rotation takes at most the whole head and needs frequencies and positions");
  if (tokens == 0) return VOSTI_OK;
  const int threads = 256;
  const size_t smem = ((size_t)2 * rot_half + (size_t)(threads / 32) * dk) * sizeof(float);
  const int r = (dk <= 128 && dv <= 128) ? 4 : 8;
  const int items = (nq + nkv) * maps + nkv + (extra_out != nullptr ? (extra_width + 32 * r - 1) / (32 * r) : 0);
  // few tokens: a warp a head; many: a block a token, so that a token's angles are formed once
  const dim3 grid(tokens, tokens < 64 ? (items + threads / 32 - 1) / (threads / 32) : 1);
#define VOSTI_HEADS_ARGS(T) proj, proj_f32, (int64_t)proj_stride, bias, (T*)q_out, (T*)k_cache, (T*)v_cache, positions, slot_mapping,  \
                            num_slots, page_size, nq, nkv, maps, dk, dv, q_norm, k_norm, norm_f32, eps, freq, rot_half, interleaved, \
                            magnitude, expanded, dk_out, dv_out, splits, plane, extra_out, extra_width, status
  if (is_f32) {
    if (r == 4) vosti_launch(qkv_heads_kernel<float, 4>, grid, dim3(threads), smem, stream, VOSTI_HEADS_ARGS(float));
    else vosti_launch(qkv_heads_kernel<float, 8>, grid, dim3(threads), smem, stream, VOSTI_HEADS_ARGS(float));
  } else {
    if (r == 4) vosti_launch(qkv_heads_kernel<bf16, 4>, grid, dim3(threads), smem, stream, VOSTI_HEADS_ARGS(bf16));
    else vosti_launch(qkv_heads_kernel<bf16, 8>, grid, dim3(threads), smem, stream, VOSTI_HEADS_ARGS(bf16));
  }
#undef VOSTI_HEADS_ARGS
  VOSTI_LAUNCH_CHECK();
}
