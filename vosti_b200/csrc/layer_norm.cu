// Layer norm (mean and variance, weight and bias) over a float32 residual stream, for blocks
// that also norm and scale what a sublayer returns before it joins the stream:
//
//   y given, with (wy, by, sy):   t = ((y - mean y) / sqrt(var y + eps_y) * wy + by) * sy
//   y given, plain:               t = y
//   x = stream + t                (stream absent: x = t)      -> stream_out (float32)
//   out = (x - mean x) / sqrt(var x + eps) * w + b            -> out (serving type or float32)
//
// so that one launch serves "norm the sublayer's output, scale it, add it, norm the sum for the
// next sublayer". The variance is the mean of the squared deviations, taken in a second walk
// over the row after the mean is known; the row lives in shared memory between the walks. All
// arithmetic is float32; reductions have a fixed order that depends on the width only.
#include "common.cuh"

namespace {

__device__ __forceinline__ float2 mean_inv(const float* row, int width, float eps, float* scratch) {
  float s = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) s += row[i];
  const float mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = row[i] - mean;
    q = fmaf(d, d, q);
  }
  const float var = block_sum(q, scratch) / (float)width;
  return make_float2(mean, 1.f / sqrtf(var + eps));
}

// Loops over a row are written in batches of U elements a thread: all loads of a batch are issued
// before its first store, because the row in shared memory, the stream and its (possibly same)
// destination are plain pointers to the compiler and a load would otherwise wait for the store
// before it, one memory latency per element.
constexpr int U = 8;

template <typename TO>
__global__ void __launch_bounds__(256)
layer_norm_stream_kernel(const float* stream, const void* y, int y_f32, const void* __restrict__ wy,
                         const void* __restrict__ by, const void* __restrict__ sy, int wy_f32, float eps_y,
                         float* stream_out, const void* __restrict__ w, const void* __restrict__ b, int w_f32, float eps,
                         TO* out, int width) {
  extern __shared__ float row[];          // [width]
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  const int step = blockDim.x;
  float2 mi = make_float2(0.f, 1.f);
  if (y != nullptr) {
    for (int i0 = threadIdx.x; i0 < width; i0 += step * U) {
      float v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = i0 + u * step < width ? load_flex(y, y_f32, base + i0 + u * step) : 0.f;
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * step < width) row[i0 + u * step] = v[u];
    }
    __syncthreads();
    if (wy != nullptr) mi = mean_inv(row, width, eps_y, scratch);
  }
  // t = the term (normed and scaled, or as it is), x = stream + t -> row, stream_out
  for (int i0 = threadIdx.x; i0 < width; i0 += step * U) {
    float t[U], a[U], c[U], e[U], x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * step;
      const bool in = i < width;
      x[u] = in && stream != nullptr ? stream[base + i] : 0.f;
      a[u] = in && wy != nullptr ? load_flex(wy, wy_f32, i) : 1.f;
      c[u] = in && wy != nullptr && by != nullptr ? load_flex(by, wy_f32, i) : 0.f;
      e[u] = in && wy != nullptr && sy != nullptr ? load_flex(sy, wy_f32, i) : 1.f;
      t[u] = in && y != nullptr ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * step;
      if (i >= width) continue;
      float term = t[u];
      if (wy != nullptr) {
        term = (term - mi.x) * mi.y * a[u];
        if (by != nullptr) term += c[u];
        if (sy != nullptr) term *= e[u];
      }
      const float sum = y == nullptr ? x[u] : stream != nullptr ? x[u] + term : term;
      row[i] = sum;
      if (stream_out != nullptr) stream_out[base + i] = sum;
    }
  }
  if (out == nullptr) return;
  __syncthreads();
  mi = mean_inv(row, width, eps, scratch);
  for (int i0 = threadIdx.x; i0 < width; i0 += step * U) {
    float a[U], c[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * step;
      a[u] = i < width ? load_flex(w, w_f32, i) : 0.f;
      c[u] = i < width && b != nullptr ? load_flex(b, w_f32, i) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * step;
      if (i < width) out[base + i] = from_f32<TO>((row[i] - mi.x) * mi.y * a[u] + c[u]);
    }
  }
}

// Four neighbouring elements of an array whose element type is chosen at run time, as one 16- or 8-byte word.
__device__ __forceinline__ float4 load4_flex(const void* p, int is_f32, int64_t quad) {
  if (is_f32) return reinterpret_cast<const float4*>(p)[quad];
  const uint2 w = reinterpret_cast<const uint2*>(p)[quad];
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&w.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void store4(float* p, int64_t quad, float4 v) { reinterpret_cast<float4*>(p)[quad] = v; }
__device__ __forceinline__ void store4(bf16* p, int64_t quad, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 w;
  w.x = *reinterpret_cast<const uint32_t*>(&lo);
  w.y = *reinterpret_cast<const uint32_t*>(&hi);
  reinterpret_cast<uint2*>(p)[quad] = w;
}

// Mean and 1 / sqrt(variance + eps) of a row held in registers, V groups of four a thread.
template <int V>
__device__ __forceinline__ float2 mean_inv_regs(const float4 (&t)[V], const bool (&in)[V], int width, float eps, float* scratch) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < V; ++j)
    if (in[j]) s += (t[j].x + t[j].y) + (t[j].z + t[j].w);
  const float mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < V; ++j)
    if (in[j]) {
      const float a = t[j].x - mean, b = t[j].y - mean, c = t[j].z - mean, d = t[j].w - mean;
      q = fmaf(a, a, q);
      q = fmaf(b, b, q);
      q = fmaf(c, c, q);
      q = fmaf(d, d, q);
    }
  const float var = block_sum(q, scratch) / (float)width;
  return make_float2(mean, 1.f / sqrtf(var + eps));
}

// The same for a width that is a multiple of four and at most 1024 V: the row stays in registers,
// every access is a 16-byte word (8 bytes for bfloat16), and everything a row needs is asked for
// before the first reduction. Which of the two kernels serves a model depends on its width only.
template <typename TO, int V>
__global__ void __launch_bounds__(256)
layer_norm_stream_vec_kernel(const float* stream, const void* y, int y_f32, const void* __restrict__ wy,
                             const void* __restrict__ by, const void* __restrict__ sy, int wy_f32, float eps_y,
                             float* stream_out, const void* __restrict__ w, const void* __restrict__ b, int w_f32, float eps,
                             TO* out, int width) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int quads = width / 4;
  const int64_t base = (int64_t)blockIdx.x * quads;
  float4 t[V], x[V];
  bool in[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int q = threadIdx.x + 256 * j;
    in[j] = q < quads;
    t[j] = in[j] && y != nullptr ? load4_flex(y, y_f32, base + q) : make_float4(0.f, 0.f, 0.f, 0.f);
    x[j] = in[j] && stream != nullptr ? reinterpret_cast<const float4*>(stream)[base + q] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (y != nullptr && wy != nullptr) {
    const float2 mi = mean_inv_regs<V>(t, in, width, eps_y, scratch);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      if (!in[j]) continue;
      const int q = threadIdx.x + 256 * j;
      const float4 a = load4_flex(wy, wy_f32, q);
      t[j] = make_float4((t[j].x - mi.x) * mi.y * a.x, (t[j].y - mi.x) * mi.y * a.y, (t[j].z - mi.x) * mi.y * a.z,
                         (t[j].w - mi.x) * mi.y * a.w);
      if (by != nullptr) {
        const float4 c = load4_flex(by, wy_f32, q);
        t[j] = make_float4(t[j].x + c.x, t[j].y + c.y, t[j].z + c.z, t[j].w + c.w);
      }
      if (sy != nullptr) {
        const float4 e = load4_flex(sy, wy_f32, q);
        t[j] = make_float4(t[j].x * e.x, t[j].y * e.y, t[j].z * e.z, t[j].w * e.w);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) {
    if (!in[j]) continue;
    if (y == nullptr) t[j] = x[j];
    else if (stream != nullptr) t[j] = make_float4(x[j].x + t[j].x, x[j].y + t[j].y, x[j].z + t[j].z, x[j].w + t[j].w);
    if (stream_out != nullptr) store4(stream_out, base + threadIdx.x + 256 * j, t[j]);
  }
  if (out == nullptr) return;
  const float2 mi = mean_inv_regs<V>(t, in, width, eps, scratch);
#pragma unroll
  for (int j = 0; j < V; ++j) {
    if (!in[j]) continue;
    const int q = threadIdx.x + 256 * j;
    const float4 a = load4_flex(w, w_f32, q);
    const float4 c = b != nullptr ? load4_flex(b, w_f32, q) : make_float4(0.f, 0.f, 0.f, 0.f);
    store4(out, base + q, make_float4((t[j].x - mi.x) * mi.y * a.x + c.x, (t[j].y - mi.x) * mi.y * a.y + c.y,
                                      (t[j].z - mi.x) * mi.y * a.z + c.z, (t[j].w - mi.x) * mi.y * a.w + c.w));
  }
}

constexpr int MAX_WIDTH = 49152;         // floats of shared memory a row may take (192 KiB)

}  // namespace

// stream: float32 [rows, width] or null; y: [rows, width] float32 or bfloat16, or null;
// wy / by / sy: the norm and the scale of y ([width], one type; wy null: y is added as it is;
// by, sy may be null); w / b: the norm of the sum (b may be null); out null: only stream_out.
VOSTI_API int vosti_layer_norm_stream(const float* stream, const void* y, int y_f32, const void* wy, const void* by,
                                      const void* sy, int wy_f32, float eps_y, float* stream_out, const void* w,
                                      const void* b, int w_f32, float eps, void* out, int out_f32, int rows, int width,
                                      cudaStream_t stream_id) {
  VOSTI_REQUIRE(rows >= 0 && width > 0 && width <= MAX_WIDTH, "layer_norm_stream: bad sizes rows=%d width=%d (at most %d)",
                rows, width, MAX_WIDTH);
  VOSTI_REQUIRE(stream != nullptr || y != nullptr, "layer_norm_stream: nothing to norm");
  VOSTI_REQUIRE(out != nullptr || stream_out != nullptr, "layer_norm_stream: nowhere to write");
  VOSTI_REQUIRE(out == nullptr || w != nullptr, "layer_norm_stream: a normed result needs a weight");
  if (rows == 0) return VOSTI_OK;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(layer_norm_stream_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_WIDTH * 4);
    cudaFuncSetAttribute(layer_norm_stream_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_WIDTH * 4);
    configured = true;
  }
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (width % 4 == 0 && width <= 8192 && aligned(stream) && aligned(y) && aligned(wy) && aligned(by) && aligned(sy) &&
      aligned(stream_out) && aligned(w) && aligned(b) && aligned(out)) {
    const int per = (width / 4 + 255) / 256;
#define VOSTI_LN_VEC(TO, V)                                                                                             \
  vosti_launch(layer_norm_stream_vec_kernel<TO, V>, dim3(rows), dim3(256), 0, stream_id, stream, y, y_f32, wy, by, sy, wy_f32, \
               eps_y, stream_out, w, b, w_f32, eps, (TO*)out, width)
#define VOSTI_LN_VEC_T(V)                                          \
  do {                                                             \
    if (out_f32) VOSTI_LN_VEC(float, V); else VOSTI_LN_VEC(bf16, V); \
  } while (0)
    if (per <= 1) VOSTI_LN_VEC_T(1);
    else if (per <= 2) VOSTI_LN_VEC_T(2);
    else if (per <= 4) VOSTI_LN_VEC_T(4);
    else VOSTI_LN_VEC_T(8);
#undef VOSTI_LN_VEC_T
#undef VOSTI_LN_VEC
    VOSTI_LAUNCH_CHECK();
  }
  const size_t smem = (size_t)width * sizeof(float);
  if (out_f32)
    vosti_launch(layer_norm_stream_kernel<float>, dim3(rows), dim3(256), smem, stream_id, stream, y, y_f32, wy, by, sy, wy_f32,
                 eps_y, stream_out, w, b, w_f32, eps, (float*)out, width);
  else
    vosti_launch(layer_norm_stream_kernel<bf16>, dim3(rows), dim3(256), smem, stream_id, stream, y, y_f32, wy, by, sy, wy_f32,
                 eps_y, stream_out, w, b, w_f32, eps, (bf16*)out, width);
  VOSTI_LAUNCH_CHECK();
}
