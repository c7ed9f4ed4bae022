// Row kernels for models that keep their residual stream in float32 whatever the serving
// type: the deferred residual sum, Dynamic Tanh (a norm without statistics), the packing of
// [stream ; first embedding] for a loop's re-entry product, and the merge of side-by-side
// mixer branches (each divided by its root mean square, weighted, averaged; or a plain sum with a
// constant per branch), the root-mean-square norm over the stream (weight stored as it is
// or around zero), and the norm after the sum of blocks that norm what they have added
// (y = rms(alpha * stream + terms) * w becomes the stream).
//
// The stream is float32 [rows, width]. A sublayer's output ("term") is float32 or the serving
// type; up to two terms wait to be added (mixer and feed-forward of a parallel block), and the
// kernel that next reads the stream adds them in a fixed order: (stream + term 1) + term 2.
#include "common.cuh"

namespace {

__device__ __forceinline__ float term_at(const void* p, int is_f32, int64_t i) {
  return p == nullptr ? 0.f : load_flex(p, is_f32, i);
}

// Four neighbouring elements starting at i (a multiple of 4) of an array whose type is chosen at
// run time: one 16-byte word of floats or one 8-byte word of bfloat16.
__device__ __forceinline__ float4 load_flex4(const void* p, int is_f32, int64_t i) {
  if (is_f32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const unsigned*>(&lo);
  raw.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// x = stream + t1 + t2 (any of them absent); stream_out <- x; out <- tanh(alpha x) * w + b.
template <typename TO>
__global__ void __launch_bounds__(256)
dyt_kernel(const float* stream, const void* t1, int t1_f32, const void* t2, int t2_f32, float* stream_out,
           const void* __restrict__ weight, const void* __restrict__ bias, int wb_f32, float alpha,
           TO* __restrict__ out, int width) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  if (width % 4 == 0) {          // the same arithmetic, four elements to a thread
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 x = stream != nullptr ? *reinterpret_cast<const float4*>(stream + base + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (t1 != nullptr) { const float4 a = load_flex4(t1, t1_f32, base + i); x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w; }
      if (t2 != nullptr) { const float4 a = load_flex4(t2, t2_f32, base + i); x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w; }
      if (stream_out != nullptr) *reinterpret_cast<float4*>(stream_out + base + i) = x;
      const float4 w = load_flex4(weight, wb_f32, i);
      float4 y = make_float4(tanhf(alpha * x.x) * w.x, tanhf(alpha * x.y) * w.y, tanhf(alpha * x.z) * w.z, tanhf(alpha * x.w) * w.w);
      if (bias != nullptr) { const float4 b = load_flex4(bias, wb_f32, i); y.x += b.x; y.y += b.y; y.z += b.z; y.w += b.w; }
      store4(out + base + i, y);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float x = stream != nullptr ? stream[base + i] : 0.f;
    if (t1 != nullptr) x += load_flex(t1, t1_f32, base + i);
    if (t2 != nullptr) x += load_flex(t2, t2_f32, base + i);
    if (stream_out != nullptr) stream_out[base + i] = x;
    float y = tanhf(alpha * x) * load_flex(weight, wb_f32, i);
    if (bias != nullptr) y += load_flex(bias, wb_f32, i);
    out[base + i] = from_f32<TO>(y);
  }
}

// out[r, 0:width] = stream + t1 + t2; out[r, width:width+tail_width] = tail[r] (optional).
template <typename TO>
__global__ void __launch_bounds__(256)
stream_sum_kernel(const float* stream, const void* t1, int t1_f32, const void* t2, int t2_f32, TO* out,
                  int64_t out_stride, const void* __restrict__ tail, int tail_f32, int tail_width, int width) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  TO* dst = out + (int64_t)blockIdx.x * out_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float x = stream != nullptr ? stream[base + i] : 0.f;
    x += term_at(t1, t1_f32, base + i);
    x += term_at(t2, t2_f32, base + i);
    dst[i] = from_f32<TO>(x);
  }
  if (tail != nullptr) {
    const int64_t tbase = (int64_t)blockIdx.x * tail_width;
    for (int i = threadIdx.x; i < tail_width; i += blockDim.x) dst[width + i] = from_f32<TO>(load_flex(tail, tail_f32, tbase + i));
  }
}

// x = stream + t1 + t2 (any of them absent); stream_out <- x; then
//   weight given:  out <- x / sqrt(mean(x^2) + eps) * (offset + weight)
//   no weight:     out <- x (rounded to the output type)
// `out` may be absent when only the sum is wanted. The row is walked twice; the second walk reads
// the sum back from stream_out where it was stored (every thread reads what it wrote itself, so
// stream_out may be the stream), else it forms the sum again from the same operands.
template <typename TO>
__global__ void __launch_bounds__(256)
rms_stream_kernel(const float* stream, const void* t1, int t1_f32, const void* t2, int t2_f32, float* stream_out,
                  const void* __restrict__ weight, int w_f32, float offset, float eps, TO* out, int width) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  const bool vec = width % 4 == 0;
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 x = stream != nullptr ? *reinterpret_cast<const float4*>(stream + base + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (t1 != nullptr) { const float4 a = load_flex4(t1, t1_f32, base + i); x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w; }
      if (t2 != nullptr) { const float4 a = load_flex4(t2, t2_f32, base + i); x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w; }
      if (stream_out != nullptr) *reinterpret_cast<float4*>(stream_out + base + i) = x;
      ss += (x.x * x.x + x.y * x.y) + (x.z * x.z + x.w * x.w);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float x = stream != nullptr ? stream[base + i] : 0.f;
      x += term_at(t1, t1_f32, base + i);
      x += term_at(t2, t2_f32, base + i);
      if (stream_out != nullptr) stream_out[base + i] = x;
      ss += x * x;
    }
  }
  if (out == nullptr) return;
  float inv = 1.f;
  if (weight != nullptr) {
    const float total = block_sum(ss, scratch);
    inv = 1.f / sqrtf(total / (float)width + eps);
  }
  if (vec) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 x;
      if (stream_out != nullptr) {
        x = *reinterpret_cast<const float4*>(stream_out + base + i);
      } else {
        x = stream != nullptr ? *reinterpret_cast<const float4*>(stream + base + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (t1 != nullptr) { const float4 a = load_flex4(t1, t1_f32, base + i); x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w; }
        if (t2 != nullptr) { const float4 a = load_flex4(t2, t2_f32, base + i); x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w; }
      }
      if (weight != nullptr) {
        const float4 w = load_flex4(weight, w_f32, i);
        x = make_float4(x.x * inv * (offset + w.x), x.y * inv * (offset + w.y), x.z * inv * (offset + w.z), x.w * inv * (offset + w.w));
      }
      store4(out + base + i, x);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float x;
    if (stream_out != nullptr) {
      x = stream_out[base + i];
    } else {
      x = stream != nullptr ? stream[base + i] : 0.f;
      x += term_at(t1, t1_f32, base + i);
      x += term_at(t2, t2_f32, base + i);
    }
    if (weight != nullptr) x = x * inv * (offset + load_flex(weight, w_f32, i));
    out[base + i] = from_f32<TO>(x);
  }
}

// Norm after the sum, for blocks that norm what they have added: s = alpha * stream + t1 + t2 in
// float32, y = s / sqrt(mean(s^2) + eps) * (offset + w); y is the new stream (float32, may be written
// over the old one: a thread writes only what it read itself) and, rounded, the next sublayer's
// input. The row is read twice, in the same order, so that any width works.
template <typename TO>
__global__ void __launch_bounds__(1024)
post_norm_stream_kernel(const float* stream, float alpha, const void* __restrict__ t1, int t1_f32, const void* __restrict__ t2,
                        int t2_f32, const void* __restrict__ weight, int w_f32, float offset, float eps, float* stream_out,
                        TO* __restrict__ out, int width, int t1_splits, int64_t t1_plane, int cached) {
  // t1_splits > 1: t1 is float32 [splits, rows, width], the unsummed K splits of a product, added in split order.
  // cached: the summed row is kept in shared memory (width floats) between the two passes; else it is formed twice.
  extern __shared__ __align__(16) float row_smem[];
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  const bool vec = width % 4 == 0;
  auto sum4 = [&](int i) {
    float4 x = *reinterpret_cast<const float4*>(stream + base + i);
    x = make_float4(x.x * alpha, x.y * alpha, x.z * alpha, x.w * alpha);
    if (t1_splits > 1) {
      // four splits' loads in flight together, added in split order
      const float* p = reinterpret_cast<const float*>(t1) + base + i;
      float4 a = *reinterpret_cast<const float4*>(p);
      int s = 1;
      for (; s + 8 <= t1_splits; s += 8) {
        float4 b[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) b[u] = *reinterpret_cast<const float4*>(p + (s + u) * t1_plane);
#pragma unroll
        for (int u = 0; u < 8; ++u) { a.x += b[u].x; a.y += b[u].y; a.z += b[u].z; a.w += b[u].w; }
      }
      for (; s + 4 <= t1_splits; s += 4) {
        const float4 b0 = *reinterpret_cast<const float4*>(p + s * t1_plane), b1 = *reinterpret_cast<const float4*>(p + (s + 1) * t1_plane);
        const float4 b2 = *reinterpret_cast<const float4*>(p + (s + 2) * t1_plane), b3 = *reinterpret_cast<const float4*>(p + (s + 3) * t1_plane);
        a.x = (((a.x + b0.x) + b1.x) + b2.x) + b3.x;
        a.y = (((a.y + b0.y) + b1.y) + b2.y) + b3.y;
        a.z = (((a.z + b0.z) + b1.z) + b2.z) + b3.z;
        a.w = (((a.w + b0.w) + b1.w) + b2.w) + b3.w;
      }
      for (; s < t1_splits; ++s) {
        const float4 b = *reinterpret_cast<const float4*>(p + s * t1_plane);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w;
    } else if (t1 != nullptr) {
      const float4 a = load_flex4(t1, t1_f32, base + i);
      x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w;
    }
    if (t2 != nullptr) { const float4 a = load_flex4(t2, t2_f32, base + i); x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w; }
    return x;
  };
  auto sum1 = [&](int i) {
    float a = term_at(t1, t1_f32, base + i);
    for (int s = 1; s < t1_splits; ++s) a += reinterpret_cast<const float*>(t1)[s * t1_plane + base + i];
    return (stream[base + i] * alpha + a) + term_at(t2, t2_f32, base + i);
  };
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      const float4 x = sum4(i);
      if (cached) *reinterpret_cast<float4*>(row_smem + i) = x;
      ss += (x.x * x.x + x.y * x.y) + (x.z * x.z + x.w * x.w);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float x = sum1(i);
      if (cached) row_smem[i] = x;
      ss += x * x;
    }
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  if (vec) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 x = cached ? *reinterpret_cast<const float4*>(row_smem + i) : sum4(i);     // (a thread reads what it wrote itself)
      const float4 w = load_flex4(weight, w_f32, i);
      x = make_float4(x.x * inv * (offset + w.x), x.y * inv * (offset + w.y), x.z * inv * (offset + w.z), x.w * inv * (offset + w.w));
      if (stream_out != nullptr) *reinterpret_cast<float4*>(stream_out + base + i) = x;
      if (out != nullptr) store4(out + base + i, x);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float x = (cached ? row_smem[i] : sum1(i)) * inv * (offset + load_flex(weight, w_f32, i));
    if (stream_out != nullptr) stream_out[base + i] = x;
    if (out != nullptr) out[base + i] = from_f32<TO>(x);
  }
}

constexpr int MAX_BRANCHES = 4;
struct Branches {
  const void* x[MAX_BRANCHES];       // [rows, width], float32 or bfloat16
  const void* w[MAX_BRANCHES];       // [width]
  int x_f32[MAX_BRANCHES];
  float scale[MAX_BRANCHES];         // the plain sum's constant per branch
  int count;
};

// out = sum_b scale_b * x_b, float32, added in branch order.
__global__ void __launch_bounds__(256)
branch_sum_kernel(Branches br, float* __restrict__ out, int width) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  if (width % 4 == 0) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int b = 0; b < br.count; ++b) {
        const float4 v = load_flex4(br.x[b], br.x_f32[b], base + i);
        const float c = br.scale[b];
        acc.x = fmaf(c, v.x, acc.x); acc.y = fmaf(c, v.y, acc.y); acc.z = fmaf(c, v.z, acc.z); acc.w = fmaf(c, v.w, acc.w);
      }
      *reinterpret_cast<float4*>(out + base + i) = acc;
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float acc = 0.f;
    for (int b = 0; b < br.count; ++b) acc = fmaf(br.scale[b], load_flex(br.x[b], br.x_f32[b], base + i), acc);
    out[base + i] = acc;
  }
}

// out = (1 / count) * sum_b  x_b / sqrt(mean(x_b^2) + eps) * w_b, float32.
__global__ void __launch_bounds__(256)
branch_merge_kernel(Branches br, int w_f32, float* __restrict__ out, int width, float eps) {
  __shared__ float scratch[32];
  __shared__ float inv_rms[MAX_BRANCHES];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  const bool vec = width % 4 == 0;
  for (int b = 0; b < br.count; ++b) {
    float ss = 0.f;
    if (vec) {
      for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
        const float4 v = load_flex4(br.x[b], br.x_f32[b], base + i);
        ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
      }
    } else {
      for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = load_flex(br.x[b], br.x_f32[b], base + i);
        ss += v * v;
      }
    }
    const float total = block_sum(ss, scratch);
    if (threadIdx.x == 0) inv_rms[b] = 1.f / sqrtf(total / (float)width + eps);
  }
  __syncthreads();
  const float share = 1.f / (float)br.count;
  if (vec) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int b = 0; b < br.count; ++b) {
        const float4 v = load_flex4(br.x[b], br.x_f32[b], base + i), w = load_flex4(br.w[b], w_f32, i);
        const float r = inv_rms[b];
        acc.x += v.x * r * w.x; acc.y += v.y * r * w.y; acc.z += v.z * r * w.z; acc.w += v.w * r * w.w;
      }
      *reinterpret_cast<float4*>(out + base + i) = make_float4(acc.x * share, acc.y * share, acc.z * share, acc.w * share);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float acc = 0.f;
    for (int b = 0; b < br.count; ++b)
      acc += load_flex(br.x[b], br.x_f32[b], base + i) * inv_rms[b] * load_flex(br.w[b], w_f32, i);
    out[base + i] = acc * share;
  }
}

}  // namespace

VOSTI_API int vosti_dyt(const float* stream, const void* t1, int t1_f32, const void* t2, int t2_f32, float* stream_out,
                        const void* weight, const void* bias, int wb_f32, float alpha, void* out, int out_f32, int rows,
                        int width, cudaStream_t stream_id) {
  VOSTI_REQUIRE(rows >= 0 && width > 0, "dyt: bad sizes rows=%d width=%d", rows, width);
  VOSTI_REQUIRE(stream != nullptr || t1 != nullptr, "dyt: nothing to norm");
  if (rows == 0) return VOSTI_OK;
  if (out_f32)
    vosti_launch(dyt_kernel<float>, dim3(rows), dim3(256), 0, stream_id, stream, t1, t1_f32, t2, t2_f32, stream_out, weight,
                 bias, wb_f32, alpha, (float*)out, width);
  else
    vosti_launch(dyt_kernel<bf16>, dim3(rows), dim3(256), 0, stream_id, stream, t1, t1_f32, t2, t2_f32, stream_out, weight,
                 bias, wb_f32, alpha, (bf16*)out, width);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_stream_sum(const float* stream, const void* t1, int t1_f32, const void* t2, int t2_f32, void* out,
                               int out_f32, int64_t out_stride, const void* tail, int tail_f32, int tail_width, int rows,
                               int width, cudaStream_t stream_id) {
  VOSTI_REQUIRE(rows >= 0 && width > 0 && out_stride >= width + (tail ? tail_width : 0),
                "stream_sum: bad sizes rows=%d width=%d", rows, width);
  if (rows == 0) return VOSTI_OK;
  if (out_f32)
    vosti_launch(stream_sum_kernel<float>, dim3(rows), dim3(256), 0, stream_id, stream, t1, t1_f32, t2, t2_f32, (float*)out,
                 out_stride, tail, tail_f32, tail_width, width);
  else
    vosti_launch(stream_sum_kernel<bf16>, dim3(rows), dim3(256), 0, stream_id, stream, t1, t1_f32, t2, t2_f32, (bf16*)out,
                 out_stride, tail, tail_f32, tail_width, width);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_branch_merge(const void* const* xs, const int* x_f32, const void* const* ws, int w_f32, int count,
                                 float* out, int rows, int width, float eps, cudaStream_t stream_id) {
  VOSTI_REQUIRE(count >= 1 && count <= MAX_BRANCHES, "branch_merge: %d branches (1 to %d are taken)", count, MAX_BRANCHES);
  VOSTI_REQUIRE(rows >= 0 && width > 0, "branch_merge: bad sizes rows=%d width=%d", rows, width);
  if (rows == 0) return VOSTI_OK;
  Branches br = {};
  br.count = count;
  for (int b = 0; b < count; ++b) {
    br.x[b] = xs[b];
    br.w[b] = ws[b];
    br.x_f32[b] = x_f32[b];
  }
  vosti_launch(branch_merge_kernel, dim3(rows), dim3(256), 0, stream_id, br, w_f32, out, width, eps);
  VOSTI_LAUNCH_CHECK();
}

// Root-mean-square norm over the float32 stream (see rms_stream_kernel); `weight` null: the sum
// alone, rounded to the output type; `out` null: only stream_out is written.
VOSTI_API int vosti_rms_stream(const float* stream, const void* t1, int t1_f32, const void* t2, int t2_f32, float* stream_out,
                               const void* weight, int w_f32, float offset, float eps, void* out, int out_f32, int rows,
                               int width, cudaStream_t stream_id) {
  VOSTI_REQUIRE(rows >= 0 && width > 0, "rms_stream: bad sizes rows=%d width=%d", rows, width);
  VOSTI_REQUIRE(stream != nullptr || t1 != nullptr, "rms_stream: nothing to norm");
  VOSTI_REQUIRE(out != nullptr || stream_out != nullptr, "rms_stream: nowhere to write");
  if (rows == 0) return VOSTI_OK;
  if (out_f32)
    vosti_launch(rms_stream_kernel<float>, dim3(rows), dim3(256), 0, stream_id, stream, t1, t1_f32, t2, t2_f32, stream_out,
                 weight, w_f32, offset, eps, (float*)out, width);
  else
    vosti_launch(rms_stream_kernel<bf16>, dim3(rows), dim3(256), 0, stream_id, stream, t1, t1_f32, t2, t2_f32, stream_out,
                 weight, w_f32, offset, eps, (bf16*)out, width);
  VOSTI_LAUNCH_CHECK();
}

// out = sum_b scales[b] * x_b, float32 [rows, width].
VOSTI_API int vosti_branch_sum(const void* const* xs, const int* x_f32, const float* scales, int count, float* out, int rows,
                               int width, cudaStream_t stream_id) {
  VOSTI_REQUIRE(count >= 1 && count <= MAX_BRANCHES, "branch_sum: %d branches (1 to %d are taken)", count, MAX_BRANCHES);
  VOSTI_REQUIRE(rows >= 0 && width > 0, "branch_sum: bad sizes rows=%d width=%d", rows, width);
  if (rows == 0) return VOSTI_OK;
  Branches br = {};
  br.count = count;
  for (int b = 0; b < count; ++b) {
    br.x[b] = xs[b];
    br.x_f32[b] = x_f32[b];
    br.scale[b] = scales[b];
  }
  vosti_launch(branch_sum_kernel, dim3(rows), dim3(256), 0, stream_id, br, out, width);
  VOSTI_LAUNCH_CHECK();
}

// Norm after the sum (see post_norm_stream_kernel): stream float32 [rows, width]; t1, t2 (either may be
// null) float32 or bfloat16, or t1 the float32 [t1_splits, rows, width] unsummed K splits of a product; stream_out float32 (may be `stream`) and / or out in the output type.
VOSTI_API int vosti_post_norm_stream(const float* stream, float alpha, const void* t1, int t1_f32, const void* t2, int t2_f32,
                                     const void* weight, int w_f32, float offset, float eps, float* stream_out, void* out,
                                     int out_f32, int rows, int width, int t1_splits, cudaStream_t stream_id) {
  VOSTI_REQUIRE(t1_splits >= 1 && (t1_splits == 1 || (t1 != nullptr && t1_f32)), "post_norm_stream: unsummed splits are float32");
  const int64_t plane = (int64_t)rows * width;
  VOSTI_REQUIRE(rows >= 0 && width > 0, "post_norm_stream: bad sizes rows=%d width=%d", rows, width);
  VOSTI_REQUIRE(stream != nullptr && weight != nullptr, "post_norm_stream: a stream and a weight are needed");
  VOSTI_REQUIRE(out != nullptr || stream_out != nullptr, "post_norm_stream: nowhere to write");
  if (rows == 0) return VOSTI_OK;
  const int cached = width <= 12288;                     // 48 KB of shared memory hold the row
  const size_t smem = cached ? (size_t)width * sizeof(float) : 0;
  // few rows: a thread a 16-byte word, so that a row's loads are all in flight at once
  int threads = 256;
  if (rows <= 64 && width % 4 == 0) threads = width / 4 >= 1024 ? 1024 : (width / 4 + 31) / 32 * 32 > 256 ? (width / 4 + 31) / 32 * 32 : 256;
  if (out_f32)
    vosti_launch(post_norm_stream_kernel<float>, dim3(rows), dim3(threads), smem, stream_id, stream, alpha, t1, t1_f32, t2, t2_f32, weight,
                 w_f32, offset, eps, stream_out, (float*)out, width, t1_splits, plane, cached);
  else
    vosti_launch(post_norm_stream_kernel<bf16>, dim3(rows), dim3(threads), smem, stream_id, stream, alpha, t1, t1_f32, t2, t2_f32, weight,
                 w_f32, offset, eps, stream_out, (bf16*)out, width, t1_splits, plane, cached);
  VOSTI_LAUNCH_CHECK();
}
