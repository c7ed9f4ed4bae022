// Latent attention on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 sums).
//
// In the latent form (see attention_latent.cu) every head of a token attends over the same keys
// [c_j | r_j] (rank + rot elements) and the same "values" c_j (rank elements): multi-query
// attention whose rows are the (token, head) pairs. A CTA takes 16 or 32 consecutive rows of one
// request (a token's heads sit next to each other, so with 16 heads a tile is one or two tokens)
// and streams the request's cached latents through shared memory in tiles of 64 keys, aligned to
// the absolute key index (cp.async straight from the pages, double-buffered):
//
//   scores   warp w of 8 takes keys 8 w .. 8 w + 7 of the tile: S = Q [rows, rank + rot] K^T
//   softmax  row maxima meet in shared memory; p = 2^(s - m) in float32; the weights go to
//            shared memory as TWO bfloat16 numbers, p = hi + lo, so that the weighted sum sees
//            16 bits of every weight's mantissa, not 8
//   sum      warp w owns the columns [w rank / 8, (w + 1) rank / 8) of the result:
//            O += (P_hi + P_lo) C, the tile's first `rank` columns read transposed by ldmatrix
//
// With few rows (decode steps) the keys are cut into segments over grid.z and every (row,
// segment) leaves (m, l, unnormalised sum) for latent_merge_kernel, like the CUDA-core kernel.
// Sizes: rank 128, 256 or 512; rot a multiple of 32; bfloat16 only. Everything else takes the
// CUDA-core kernel.
#include "common.cuh"
#include "mma_util.cuh"

namespace {

constexpr int LW = 8;              // warps of a CTA
constexpr int LKT = 64;            // keys of a tile
constexpr int P_PITCH = LKT * 2 + 16;
constexpr float LOG2E = 1.4426950408889634f;

template <int RANK, int MT, int HALVES>
__global__ void __launch_bounds__(LW * HALVES * 32, 1)
latent_attend_mma_kernel(const bf16* __restrict__ qk, const bf16* __restrict__ c_cache, const bf16* __restrict__ r_cache,
                         float* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ cu_q,
                         const int* __restrict__ block_table, int max_pages, int page_size, int num_pages, int heads,
                         int rot, float scale_log2, int window, float* __restrict__ partial, int segment,
                         unsigned* status) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_wait();
  pdl_launch_dependents();
  constexpr int ROWS = 16 * MT * HALVES;         // HALVES groups of LW warps, each with MT row tiles of its own
  constexpr int NW = LW * HALVES;
  constexpr int NT = RANK / (8 * LW);            // 8-column tiles of the result a warp owns
  const int lane = threadIdx.x & 31, warp_all = threadIdx.x >> 5;
  const int warp = warp_all % LW, half_row = (warp_all / LW) * 16 * MT;     // the group's first row of the tile
  const int b = blockIdx.y;
  const int q_start = cu_q[b], q_len = cu_q[b + 1] - q_start;
  const int rows_total = q_len * heads;
  const int row0 = blockIdx.x * ROWS;
  if (row0 >= rows_total) return;
  const int kw = RANK + rot;
  const int pitch = kw * 2 + 16;                 // an odd number of 16-byte words: ldmatrix rows fall into different banks
  const int chunks = kw / 8;
  uint8_t* q_s = smem;                                      // [ROWS][pitch]
  uint8_t* k_s = q_s + ROWS * pitch;                        // 2 x [LKT][pitch]
  uint8_t* p_s = k_s + 2 * LKT * pitch;                     // 2 (hi, lo) x [ROWS][P_PITCH]
  float* red_s = reinterpret_cast<float*>(p_s + 2 * ROWS * P_PITCH);       // [LW][ROWS]

  const int64_t first_row = (int64_t)q_start * heads + row0;                // in [tokens * heads]
  for (int i = threadIdx.x; i < ROWS * chunks; i += NW * 32) {
    const int r = i / chunks, c = i % chunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row0 + r < rows_total) v = *reinterpret_cast<const uint4*>(qk + (first_row + r) * kw + c * 8);
    *reinterpret_cast<uint4*>(q_s + r * pitch + c * 16) = v;
  }

  // this thread's rows: (lane / 4) + 8 r of each 16-row tile
  int pos_row[MT][2], kstart_row[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int packed = row0 + half_row + mt * 16 + (lane >> 2) + 8 * r;
      pos_row[mt][r] = packed < rows_total ? positions[q_start + packed / heads] : -1;     // -1: sees nothing, writes nothing
      kstart_row[mt][r] = pos_row[mt][r] >= 0 ? first_visible_key(pos_row[mt][r], window) : 0;
    }
  const int token_lo = row0 / heads, token_hi = min(q_len - 1, (row0 + ROWS - 1) / heads);
  const int pos_lo = positions[q_start + token_lo], pos_hi = positions[q_start + token_hi];
  int first_key = first_visible_key(pos_lo, window), key_end = pos_hi + 1;   // [first_key, key_end)
  if (partial != nullptr) {
    first_key = max(first_key, (int)blockIdx.z * segment);
    key_end = min(key_end, (int)(blockIdx.z + 1) * segment);
  }
  const int segments = gridDim.z;
  if (first_key >= key_end) {                    // nothing of this segment is visible: empty records
    if (partial != nullptr)
      for (int r = threadIdx.x; r < ROWS && row0 + r < rows_total; r += NW * 32) {
        float* rec = partial + ((first_row + r) * segments + blockIdx.z) * (int64_t)(RANK + 2);
        rec[0] = -INFINITY;
        rec[1] = 0.f;
      }
    return;
  }
  const int tile_begin = (first_key / LKT) * LKT;
  const int tiles = (key_end - tile_begin + LKT - 1) / LKT;
  const int* table = block_table + (int64_t)b * max_pages;
  const int rank_chunks = RANK / 8;

  auto issue = [&](int tile, int buffer) {
    const int key0 = tile_begin + tile * LKT;
    uint8_t* dst = k_s + buffer * (LKT * pitch);
    // lane i looks up the slot of the warp's i-th row; the rows then take it from there
    int64_t my_slot = -1;
    if (lane < LKT / NW) {
      const int key = key0 + warp_all + lane * NW;
      if (key >= first_key && key < key_end) {
        const int index = key / page_size;
        const int page = index < max_pages ? table[index] : -1;
        if (page < 0 || page >= num_pages) raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
        else my_slot = (int64_t)page * page_size + (key - index * page_size);
      }
    }
#pragma unroll
    for (int i = 0; i < LKT / NW; ++i) {
      const int r = warp_all + i * NW;
      int64_t slot = __shfl_sync(0xffffffffu, my_slot, i);
      const bool valid = slot >= 0;
      if (!valid) slot = 0;
      const bf16* crow = c_cache + slot * RANK;
      const bf16* rrow = r_cache + slot * rot;
      for (int c = lane; c < chunks; c += 32) {
        if (valid) cp_async16(smem_addr(dst + r * pitch + c * 16), c < rank_chunks ? crow + c * 8 : rrow + (c - rank_chunks) * 8);
        else *reinterpret_cast<uint4*>(dst + r * pitch + c * 16) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };

  float m_row[MT][2], l_row[MT][2];
  float o[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_row[mt][0] = m_row[mt][1] = -INFINITY;
    l_row[mt][0] = l_row[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < NT; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
  }
  const int col0 = warp * (RANK / LW);           // the warp's first column of the result

  issue(0, 0);
  for (int tile = 0; tile < tiles; ++tile) {
    const int buffer = tile & 1;
    if (tile + 1 < tiles) {
      issue(tile + 1, buffer ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint8_t* ks = k_s + buffer * (LKT * pitch);
    const int key0 = tile_begin + tile * LKT;

    // ---- scores of the warp's 8 keys against all rows
    // four separate running sums a row tile (two per step, alternating steps), so that an mma does not wait
    // for the one before it; they meet once the key is through
    float s[MT][4], sa[MT][4], sb[MT][4], sc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[mt][e] = sa[mt][e] = sb[mt][e] = sc[mt][e] = 0.f;
    const uint32_t k_lane = smem_addr(ks + (warp * 8 + (lane & 7)) * pitch + (lane >> 3) * 16);
    const uint32_t q_lane = smem_addr(q_s + (half_row + (lane & 15)) * pitch + (lane >> 4) * 16);
    auto step = [&](int kk, float (&first)[MT][4], float (&second)[MT][4]) {       // 32 elements of the key: two mma k-steps
      uint32_t bm[4];
      ldmatrix_x4(bm, k_lane + kk * 64);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a[4], a2[4];
        ldmatrix_x4(a, q_lane + mt * 16 * pitch + kk * 64);
        ldmatrix_x4(a2, q_lane + mt * 16 * pitch + kk * 64 + 32);
        mma_bf16(first[mt], a, bm[0], bm[1]);
        mma_bf16(second[mt], a2, bm[2], bm[3]);
      }
    };
    const int key_steps = kw / 32;
    int kk = 0;
    for (; kk + 1 < key_steps; kk += 2) {
      step(kk, s, sa);
      step(kk + 1, sb, sc);
    }
    if (kk < key_steps) step(kk, s, sa);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[mt][e] = (s[mt][e] + sa[mt][e]) + (sb[mt][e] + sc[mt][e]);
    // ---- mask, scale, the tile's row maxima across the warps
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + warp * 8 + (lane & 3) * 2 + (e & 1);
        const int r = e >> 1;
        const bool visible = key <= pos_row[mt][r] && key >= kstart_row[mt][r] && key >= first_key && key < key_end;
        s[mt][e] = visible ? s[mt][e] * scale_log2 : -INFINITY;
        tile_max[r] = fmaxf(tile_max[r], s[mt][e]);
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        if ((lane & 3) == 0) red_s[warp * ROWS + half_row + mt * 16 + (lane >> 2) + 8 * r] = tile_max[r];
      }
    }
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = half_row + mt * 16 + (lane >> 2) + 8 * r;
        float tile_max = -INFINITY;
#pragma unroll
        for (int w = 0; w < LW; ++w) tile_max = fmaxf(tile_max, red_s[w * ROWS + row]);
        const float m_new = fmaxf(m_row[mt][r], tile_max);
        const float safe = m_new == -INFINITY ? 0.f : m_new;
        alpha[r] = fast_exp2(m_row[mt][r] - safe);
        m_row[mt][r] = m_new;
        const float p0 = fast_exp2(s[mt][2 * r] - safe), p1 = fast_exp2(s[mt][2 * r + 1] - safe);
        l_row[mt][r] = l_row[mt][r] * alpha[r] + p0 + p1;              // this thread's keys only; joined at the end
        const __nv_bfloat162 hi = __floats2bfloat162_rn(p0, p1);
        const float2 back = __bfloat1622float2(hi);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(p0 - back.x, p1 - back.y);
        uint8_t* at = p_s + row * P_PITCH + (warp * 8 + (lane & 3) * 2) * 2;
        *reinterpret_cast<__nv_bfloat162*>(at) = hi;
        *reinterpret_cast<__nv_bfloat162*>(at + ROWS * P_PITCH) = lo;
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        o[mt][nt][0] *= alpha[0]; o[mt][nt][1] *= alpha[0];
        o[mt][nt][2] *= alpha[1]; o[mt][nt][3] *= alpha[1];
      }
    }
    __syncthreads();
    // ---- O += (P_hi + P_lo) C over the warp's columns, 16 keys at a time
    const uint32_t p_lane = smem_addr(p_s + (half_row + (lane & 15)) * P_PITCH + (lane >> 4) * 16);
    const uint32_t v_lane = smem_addr(ks + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (col0 + (lane >> 4) * 8) * 2);
#pragma unroll
    for (int j = 0; j < LKT / 16; ++j) {
      if (key0 + j * 16 >= key_end) break;
      uint32_t hi[MT][4], lo[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        ldmatrix_x4(hi[mt], p_lane + mt * 16 * P_PITCH + j * 32);
        ldmatrix_x4(lo[mt], p_lane + (ROWS + mt * 16) * P_PITCH + j * 32);
      }
      // all the warp's column tiles with the leading terms first, then with the remainders: an mma never
      // follows another on the same sums
      uint32_t bm[NT / 2][4];
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) ldmatrix_x4_trans(bm[n2], v_lane + j * 16 * pitch + n2 * 32);
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(o[mt][2 * n2], hi[mt], bm[n2][0], bm[n2][1]);
          mma_bf16(o[mt][2 * n2 + 1], hi[mt], bm[n2][2], bm[n2][3]);
        }
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(o[mt][2 * n2], lo[mt], bm[n2][0], bm[n2][1]);
          mma_bf16(o[mt][2 * n2 + 1], lo[mt], bm[n2][2], bm[n2][3]);
        }
    }
    __syncthreads();          // everyone is done with this buffer, the weights and the maxima
  }

  // ---- the rows' sums of weights: over the thread's quad, then over the warps
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_row[mt][r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if ((lane & 3) == 0) red_s[warp * ROWS + half_row + mt * 16 + (lane >> 2) + 8 * r] = l;
    }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (pos_row[mt][r] < 0) continue;
      const int row = half_row + mt * 16 + (lane >> 2) + 8 * r;
      float l = 0.f;
#pragma unroll
      for (int w = 0; w < LW; ++w) l += red_s[w * ROWS + row];
      float* dst;
      float inv = 1.f;
      if (partial != nullptr) {
        float* rec = partial + ((first_row + row) * segments + blockIdx.z) * (int64_t)(RANK + 2);
        if (warp == 0 && (lane & 3) == 0) {
          rec[0] = m_row[mt][r];
          rec[1] = l;
        }
        dst = rec + 2;
      } else {
        dst = out + (first_row + row) * RANK;
        inv = l > 0.f ? 1.f / l : 0.f;
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        *reinterpret_cast<float2*>(dst + col0 + nt * 8 + (lane & 3) * 2) =
            make_float2(o[mt][nt][2 * r] * inv, o[mt][nt][2 * r + 1] * inv);
    }
}

__device__ __forceinline__ void store_pair(float* at, float a, float b) { *reinterpret_cast<float2*>(at) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* at, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(at) = __floats2bfloat162_rn(a, b); }

// ---- y[t, h, :] = g[t, h] * (x[t, h, :] @ M_h) on the tensor cores: one small product per head.
// A CTA takes 16 WM tokens x 8 NT WN outputs of one head; the inner extent passes through shared
// memory 64 elements at a time while the next piece is already on its way in registers. M_h is
// read where it lies: rows of outputs with the inner index contiguous (KMAJOR) or rows of inner
// elements with the output index contiguous. A float32 x enters as two bfloat16 terms, x = hi + lo,
// so that the product sees 16 bits of its mantissa.
constexpr int HPK = 64;

template <bool XF32, bool KMAJOR, int WM, int WN, int NT, typename TY>
__global__ void __launch_bounds__(WM * WN * 32)
head_project_mma_kernel(const void* __restrict__ x_, int64_t x_row, int64_t x_head, const bf16* __restrict__ m,
                        int64_t m_head, int64_t m_stride, const float* __restrict__ gate, TY* __restrict__ y,
                        int64_t y_row, int64_t y_head, int tokens, int heads, int in, int out) {
  constexpr int THREADS = WM * WN * 32, TM = 16 * WM, TN = 8 * NT * WN;
  constexpr int A_PITCH = HPK + 8;
  constexpr int B_ROWS = KMAJOR ? TN : HPK, B_COLS = KMAJOR ? HPK : TN, B_PITCH = B_COLS + 8;
  constexpr int AV = TM * (HPK / 8) / THREADS, BV = B_ROWS * (B_COLS / 8) / THREADS;
  static_assert(AV >= 1 && BV >= 1 && NT % 2 == 0, "head_project_mma: tile shape");
  __shared__ __align__(16) bf16 a_s[XF32 ? 2 : 1][TM][A_PITCH];
  __shared__ __align__(16) bf16 b_s[B_ROWS][B_PITCH];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp % WM, wn = warp / WM;
  const int h = blockIdx.y, t0 = blockIdx.z * TM, o0 = blockIdx.x * TN;
  const bf16* mh = m + (int64_t)h * m_head;

  uint4 a_reg[AV][XF32 ? 2 : 1], b_reg[BV];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int v = 0; v < AV; ++v) {
      const int idx = tid + v * THREADS, r = idx / (HPK / 8), c = idx % (HPK / 8);
      const int t = t0 + r, k = k0 + c * 8;
      const bool valid = t < tokens && k < in;
      if (XF32) {
        const float* src = reinterpret_cast<const float*>(x_) + (int64_t)t * x_row + (int64_t)h * x_head + k;
        a_reg[v][0] = valid ? *reinterpret_cast<const uint4*>(src) : make_uint4(0, 0, 0, 0);
        a_reg[v][XF32 ? 1 : 0] = valid ? *reinterpret_cast<const uint4*>(src + 4) : make_uint4(0, 0, 0, 0);
      } else {
        const bf16* src = reinterpret_cast<const bf16*>(x_) + (int64_t)t * x_row + (int64_t)h * x_head + k;
        a_reg[v][0] = valid ? *reinterpret_cast<const uint4*>(src) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int v = 0; v < BV; ++v) {
      const int idx = tid + v * THREADS, r = idx / (B_COLS / 8), c = idx % (B_COLS / 8);
      const int k = KMAJOR ? k0 + c * 8 : k0 + r, o = KMAJOR ? o0 + r : o0 + c * 8;
      const bf16* src = mh + (KMAJOR ? (int64_t)o * m_stride + k : (int64_t)k * m_stride + o);
      b_reg[v] = (k < in && o < out) ? *reinterpret_cast<const uint4*>(src) : make_uint4(0, 0, 0, 0);
    }
  };
  auto stage = [&]() {
#pragma unroll
    for (int v = 0; v < AV; ++v) {
      const int idx = tid + v * THREADS, r = idx / (HPK / 8), c = idx % (HPK / 8);
      if (XF32) {
        const float* f0 = reinterpret_cast<const float*>(&a_reg[v][0]);
        const float* f1 = reinterpret_cast<const float*>(&a_reg[v][XF32 ? 1 : 0]);
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float u0 = e < 2 ? f0[2 * e] : f1[2 * e - 4], u1 = e < 2 ? f0[2 * e + 1] : f1[2 * e - 3];
          const __nv_bfloat162 top = __floats2bfloat162_rn(u0, u1);
          const float2 back = __bfloat1622float2(top);
          hi[e] = *reinterpret_cast<const uint32_t*>(&top);
          lo[e] = pack_bf16(u0 - back.x, u1 - back.y);
        }
        *reinterpret_cast<uint4*>(&a_s[0][r][c * 8]) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(&a_s[XF32 ? 1 : 0][r][c * 8]) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      } else {
        *reinterpret_cast<uint4*>(&a_s[0][r][c * 8]) = a_reg[v][0];
      }
    }
#pragma unroll
    for (int v = 0; v < BV; ++v) {
      const int idx = tid + v * THREADS, r = idx / (B_COLS / 8), c = idx % (B_COLS / 8);
      *reinterpret_cast<uint4*>(&b_s[r][c * 8]) = b_reg[v];
    }
  };

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  const int n_warp = wn * NT * 8;                // the warp's first output column of the tile

  fetch(0);
  for (int k0 = 0; k0 < in; k0 += HPK) {
    __syncthreads();
    stage();
    __syncthreads();
    if (k0 + HPK < in) fetch(k0 + HPK);
#pragma unroll
    for (int kk = 0; kk < HPK / 32; ++kk) {      // 32 inner elements a step: two mma k-steps
      uint32_t a_hi[2][4], a_lo[2][4];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        ldmatrix_x4(a_hi[s], smem_addr(&a_s[0][wm * 16 + (lane & 15)][kk * 32 + s * 16 + (lane >> 4) * 8]));
        if (XF32) ldmatrix_x4(a_lo[s], smem_addr(&a_s[XF32 ? 1 : 0][wm * 16 + (lane & 15)][kk * 32 + s * 16 + (lane >> 4) * 8]));
      }
      if (KMAJOR) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint32_t bm[4];
          ldmatrix_x4(bm, smem_addr(&b_s[n_warp + nt * 8 + (lane & 7)][kk * 32 + (lane >> 3) * 8]));
          mma_bf16(acc[nt], a_hi[0], bm[0], bm[1]);
          mma_bf16(acc[nt], a_hi[1], bm[2], bm[3]);
          if (XF32) {
            mma_bf16(acc[nt], a_lo[0], bm[0], bm[1]);
            mma_bf16(acc[nt], a_lo[1], bm[2], bm[3]);
          }
        }
      } else {
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int n2 = 0; n2 < NT / 2; ++n2) {
            uint32_t bm[4];
            ldmatrix_x4_trans(bm, smem_addr(&b_s[kk * 32 + s * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][n_warp + n2 * 16 + (lane >> 4) * 8]));
            mma_bf16(acc[2 * n2], a_hi[s], bm[0], bm[1]);
            mma_bf16(acc[2 * n2 + 1], a_hi[s], bm[2], bm[3]);
            if (XF32) {
              mma_bf16(acc[2 * n2], a_lo[s], bm[0], bm[1]);
              mma_bf16(acc[2 * n2 + 1], a_lo[s], bm[2], bm[3]);
            }
          }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int t = t0 + wm * 16 + (lane >> 2) + 8 * r;
    if (t >= tokens) continue;
    const float g = gate != nullptr ? gate[(int64_t)t * heads + h] : 1.f;
    TY* dst = y + (int64_t)t * y_row + (int64_t)h * y_head;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int o = o0 + n_warp + nt * 8 + (lane & 3) * 2;
      if (o >= out) continue;
      store_pair(dst + o, acc[nt][2 * r] * g, acc[nt][2 * r + 1] * g);
    }
  }
}

size_t latent_mma_smem(int rank, int rot, int rows) {
  const size_t pitch = (size_t)(rank + rot) * 2 + 16;
  return (rows + 2 * LKT) * pitch + 2 * rows * P_PITCH + LW * rows * sizeof(float);
}

}  // namespace

// 1 if the tensor-core kernel takes these sizes (bfloat16 is the caller's to check).
VOSTI_API int vosti_latent_attend_mma_fits(int rank, int rot) {
  return (rank == 128 || rank == 256 || rank == 512) && rot > 0 && rot % 32 == 0 && latent_mma_smem(rank, rot, 32) <= 227 * 1024;
}

// qk bf16 [tokens, heads, rank + rot]; caches bf16 [pages, 1, page_size, rank | rot]; out float32
// [tokens, heads, rank]. Serves requests 0 .. requests - 1 of cu_q, the longest portion having
// max_q_len tokens. With `segments` > 1 the keys are cut into pieces of `segment` keys (a multiple
// of 64) and `scratch` holds tokens * heads * segments * (rank + 2) floats for latent_merge.
VOSTI_API int vosti_latent_attend_mma(const void* qk, const void* c_cache, const void* r_cache, float* out,
                                      const int* positions, const int* cu_q, const int* block_table, int max_pages,
                                      int page_size, int num_pages, int requests, int max_q_len, int heads, int rank,
                                      int rot, float scale, int window, float* scratch, int segment, int segments,
                                      unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(vosti_latent_attend_mma_fits(rank, rot), "latent_attend_mma: rank %d, rot %d are not sizes this kernel takes", rank, rot);
  VOSTI_REQUIRE(requests >= 0 && requests <= 65535 && heads > 0 && max_q_len >= 0, "latent_attend_mma: bad sizes");
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "latent_attend_mma: bad cache geometry");
  VOSTI_REQUIRE(segments >= 1 && segments <= 65535 && (segments == 1 || (scratch != nullptr && segment > 0 && segment % LKT == 0)),
                "latent_attend_mma: key segments need scratch and a length that is a multiple of %d", LKT);
  if (requests == 0 || max_q_len == 0) return VOSTI_OK;
  const int64_t most_rows = (int64_t)max_q_len * heads;
  const int halves = most_rows > 16 ? 2 : 1;      // 32 rows: two groups of warps with a row tile each over the same keys
  const int rows = 16 * halves;
  const int64_t tiles = (most_rows + rows - 1) / rows;
  VOSTI_REQUIRE(tiles <= 0x7fffffffLL, "latent_attend_mma: too many rows");
  const dim3 grid((unsigned)tiles, requests, segments);
  const size_t smem = latent_mma_smem(rank, rot, rows);
  float* partial = segments > 1 ? scratch : nullptr;
#define VOSTI_LM(RANK, HALVES)                                                                                          \
  do {                                                                                                                  \
    static bool configured = false;                                                                                     \
    if (!configured) {                                                                                                  \
      cudaFuncSetAttribute(latent_attend_mma_kernel<RANK, 1, HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); \
      configured = true;                                                                                                \
    }                                                                                                                   \
    vosti_launch(latent_attend_mma_kernel<RANK, 1, HALVES>, grid, dim3(LW * HALVES * 32), smem, stream, (const bf16*)qk, \
                 (const bf16*)c_cache, (const bf16*)r_cache, out, positions, cu_q, block_table, max_pages, page_size,   \
                 num_pages, heads, rot, scale * LOG2E, window, partial, segment, status);                               \
  } while (0)
  if (rank == 512) { if (halves == 2) VOSTI_LM(512, 2); else VOSTI_LM(512, 1); }
  else if (rank == 256) { if (halves == 2) VOSTI_LM(256, 2); else VOSTI_LM(256, 1); }
  else { if (halves == 2) VOSTI_LM(128, 2); else VOSTI_LM(128, 1); }
#undef VOSTI_LM
  VOSTI_LAUNCH_CHECK();
}

// y[t, h, o] = gate[t, h] * sum_i x[t, h, i] * m[h * m_head + i * m_in + o * m_out] with a bfloat16 m
// whose inner or output index is contiguous (m_in == 1 or m_out == 1), on the tensor cores. The
// caller has checked vosti_head_project_mma_fits. x and y float32 or bfloat16; strides in elements.
VOSTI_API int vosti_head_project_mma_fits(int64_t x_row, int64_t x_head, int x_f32, int64_t m_head, int64_t m_in,
                                          int64_t m_out, int64_t y_row, int64_t y_head, int in, int out) {
  const int xv = x_f32 ? 4 : 8;
  const int64_t m_stride = m_in == 1 ? m_out : m_in;
  return (m_in == 1 || m_out == 1) && in % 8 == 0 && out % 8 == 0 && x_row % xv == 0 && x_head % xv == 0 &&
         m_head % 8 == 0 && m_stride % 8 == 0 && y_row % 2 == 0 && y_head % 2 == 0;
}

VOSTI_API int vosti_head_project_mma(const void* x, int x_f32, int64_t x_row, int64_t x_head, const void* m,
                                     int64_t m_head, int64_t m_in, int64_t m_out, const float* gate, void* y, int y_f32,
                                     int64_t y_row, int64_t y_head, int tokens, int heads, int in, int out,
                                     cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && heads > 0 && heads <= 65535 && in > 0 && out > 0, "head_project_mma: bad sizes");
  VOSTI_REQUIRE(vosti_head_project_mma_fits(x_row, x_head, x_f32, m_head, m_in, m_out, y_row, y_head, in, out),
                "head_project_mma: strides or sizes this kernel does not take");
  VOSTI_REQUIRE((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(m)) % 16 == 0 &&
                reinterpret_cast<uintptr_t>(y) % 8 == 0, "head_project_mma: operands are not aligned");
  if (tokens == 0) return VOSTI_OK;
  const bool kmajor = m_in == 1;
  const int64_t m_stride = kmajor ? m_out : m_in;
  const bool few = tokens <= 16;
  const int tm = few ? 16 : 64, tn = few ? 64 : 128;
  const int token_tiles = (tokens + tm - 1) / tm;
  VOSTI_REQUIRE(token_tiles <= 65535, "head_project_mma: too many tokens for one launch");
  const dim3 grid((out + tn - 1) / tn, heads, token_tiles);
#define VOSTI_HPM(XF, KM, WM, WN, NT, TY)                                                                          \
  vosti_launch(head_project_mma_kernel<XF, KM, WM, WN, NT, TY>, grid, dim3(WM * WN * 32), 0, stream, x, x_row,     \
               x_head, (const bf16*)m, m_head, m_stride, gate, (TY*)y, y_row, y_head, tokens, heads, in, out)
#define VOSTI_HPM_SHAPE(XF, KM, TY)                                                                                \
  do {                                                                                                             \
    if (few) VOSTI_HPM(XF, KM, 1, 4, 2, TY);                                                                       \
    else VOSTI_HPM(XF, KM, 4, 2, 8, TY);                                                                           \
  } while (0)
#define VOSTI_HPM_TYPES(XF, KM)                                                                                    \
  do {                                                                                                             \
    if (y_f32) VOSTI_HPM_SHAPE(XF, KM, float);                                                                     \
    else VOSTI_HPM_SHAPE(XF, KM, bf16);                                                                            \
  } while (0)
  if (x_f32) { if (kmajor) VOSTI_HPM_TYPES(true, true); else VOSTI_HPM_TYPES(true, false); }
  else { if (kmajor) VOSTI_HPM_TYPES(false, true); else VOSTI_HPM_TYPES(false, false); }
#undef VOSTI_HPM_TYPES
#undef VOSTI_HPM_SHAPE
#undef VOSTI_HPM
  VOSTI_LAUNCH_CHECK();
}
