// kq_idot — the integer-dot ("i8a8") form of the quantized linear: per-token int8
// activations against resident int8 (w8a8) or int4 (w4a8) weights.
//
// Replaces packages/runtime/src/kernels/quantize-rows.ts:83-155 (activation quantisation)
// and packages/runtime/src/kernels/linear-i8a8.ts:21-72 (the two integer GEMM variants); the
// CPU statement of the same contracts is packages/runtime/src/reference/i8a8.ts:87-229.
//
// Numeric contracts (integer sums are exact, so every implementation reaches the same bits):
//   quantize_rows : s = max(amax(|x|) * (1/127), f32 tiny) with NaN propagated into s;
//                   q = clamp(round_ties_even(x / s), -127, 127), IEEE division
//   w8a8          : out = fma(f32(sum_k xq*wq), fround(xs[row] * ws[col]), bias[col])
//   w4a8          : accf = 0; per group, ascending: accf = fma(f32(sum_{k in g} xq*wq), ws[col,g], accf);
//                   out = fma(accf, xs[row], bias[col])
//
// Two kernels per variant: a generic one (any layout, any legal shape: one thread per
// output) and a tensor-core one for the library's tiled layouts, where the stored bytes ARE
// the A fragment of mma.sync.m16n8k32 (int8: q + 128 as u8, no unpack at all; int4: two
// masks and a shift per 8 weights) and the stored offset is taken out as an exact integer
// correction (128 * sum xq per row, 8 * sum xq per group).
#include <algorithm>
#include <type_traits>

#include "kq_common.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr float kInv127 = static_cast<float>(1.0 / 127.0);
constexpr float kF32Tiny = 1.1754943508222875e-38f;

__device__ __forceinline__ bool is_nan_bits(float v) { return (__float_as_uint(v) & 0x7fffffffu) > 0x7f800000u; }

// One CTA per row.  Writes q[row, dim] (int8), scale[row], and the integer sums the
// tensor-core kernels subtract: row_sum[row] = sum q, group_sum[row, dim/32] = sum q over each
// 32-element group (written only when dim % 32 == 0).
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const float* __restrict__ x, uint32_t rows, uint32_t dim, int8_t* __restrict__ q,
                     float* __restrict__ scale, int* __restrict__ row_sum, int* __restrict__ group_sum) {
  __shared__ float s_max[8];
  __shared__ int s_nan[8];
  __shared__ int s_sum[8];
  __shared__ float s_scale;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + static_cast<size_t>(row) * dim;
    float amax = 0.0f;
    int saw_nan = 0;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
      const float v = fabsf(xr[i]);
      if (is_nan_bits(v)) saw_nan = 1;
      else amax = fmaxf(amax, v);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
      saw_nan |= __shfl_xor_sync(0xffffffffu, saw_nan, off);
    }
    if (lane == 0) {
      s_max[warp] = amax;
      s_nan[warp] = saw_nan;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.0f;
      int nan = 0;
      for (uint32_t w = 0; w < blockDim.x / 32; ++w) {
        a = fmaxf(a, s_max[w]);
        nan |= s_nan[w];
      }
      float s = __fmul_rn(a, kInv127);
      if (s < kF32Tiny) s = kF32Tiny;
      if (nan) s = __int_as_float(0x7fc00000);
      s_scale = s;
      scale[row] = s;
    }
    __syncthreads();
    const float s = s_scale;
    int local = 0;
    const uint32_t groups = dim / 32;
    const bool want_groups = group_sum != nullptr && dim % 32 == 0;
    // consecutive threads take consecutive elements, so a warp covers exactly one 32-group per pass
    for (uint32_t i = threadIdx.x; i < ((dim + 31u) & ~31u); i += blockDim.x) {
      int v = 0;
      if (i < dim) {
        float r = rintf(__fdiv_rn(xr[i], s));
        if (!(r >= -127.0f)) r = -127.0f;  // also gives NaN, outside the contract, a fixed value
        if (r > 127.0f) r = 127.0f;
        v = static_cast<int>(r);
        q[static_cast<size_t>(row) * dim + i] = static_cast<int8_t>(v);
      }
      int gs = v;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) gs += __shfl_xor_sync(0xffffffffu, gs, off);
      if (want_groups && lane == 0 && i < dim) group_sum[static_cast<size_t>(row) * groups + (i >> 5)] = gs;
      if (lane == 0) local += gs;
    }
    if (lane == 0) s_sum[warp] = local;
    __syncthreads();
    if (threadIdx.x == 0 && row_sum != nullptr) {
      int total = 0;
      for (uint32_t w = 0; w < blockDim.x / 32; ++w) total += s_sum[w];
      row_sum[row] = total;
    }
    __syncthreads();
  }
}

// Integer sums of already-quantised activations (what quantize_rows_kernel also produces):
// one warp per 32-element group, one CTA per row.
__global__ void __launch_bounds__(256)
xq_sums_kernel(const int8_t* __restrict__ q, uint32_t rows, uint32_t dim, int* __restrict__ row_sum,
               int* __restrict__ group_sum) {
  __shared__ int s_sum[8];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t row = blockIdx.x;
  const uint32_t groups = dim / 32;
  const bool want_groups = dim % 32 == 0;
  int local = 0;
  for (uint32_t i = threadIdx.x; i < ((dim + 31u) & ~31u); i += blockDim.x) {
    int gs = i < dim ? static_cast<int>(q[static_cast<size_t>(row) * dim + i]) : 0;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) gs += __shfl_xor_sync(0xffffffffu, gs, off);
    if (want_groups && lane == 0 && i < dim) group_sum[static_cast<size_t>(row) * groups + (i >> 5)] = gs;
    if (lane == 0) local += gs;
  }
  if (lane == 0) s_sum[warp] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0;
    for (uint32_t w = 0; w < blockDim.x / 32; ++w) total += s_sum[w];
    row_sum[row] = total;
  }
}

// ---- generic integer-dot linear: one thread per output, any layout --------------------------
struct IdotParams {
  const uint8_t* w;      // payload (native) or tiled chunks
  const void* scale;     // native: scales; tiled int8: scales; tiled int4: nullptr (inside the chunks)
  int layout, storage, scale_f16;
  uint32_t n, k, group_size;
  const int8_t* xq;
  const float* xs;
  const float* bias;
  float* out;
  uint32_t m;
};

__device__ __forceinline__ int weight_q(const IdotParams& p, uint32_t col, uint32_t kk) {
  if (p.storage == KQ_STORAGE_I8) {
    if (p.layout == kLayoutTiledI8) return static_cast<int>(p.w[tiled_i8_locate(col, kk, p.k)]) - 128;
    return static_cast<int>(reinterpret_cast<const int8_t*>(p.w)[static_cast<size_t>(col) * p.k + kk]);
  }
  if (p.layout == kLayoutTiledI4) {
    const TiledPos pos = tiled_i4_locate(col, kk, p.k, p.scale_f16 ? 2u : 4u);
    const uint32_t word = *reinterpret_cast<const uint32_t*>(p.w + pos.word_offset);
    return static_cast<int>((word >> (4u * pos.nibble)) & 15u) - 8;
  }
  const size_t flat = static_cast<size_t>(col) * p.k + kk;
  const uint32_t byte = p.w[flat >> 1];
  return static_cast<int>((flat & 1u) ? (byte >> 4) : (byte & 15u)) - 8;
}

__device__ __forceinline__ float weight_scale(const IdotParams& p, uint32_t col, uint32_t group) {
  if (p.storage == KQ_STORAGE_I8)
    return p.scale_f16 ? load_scale<true>(p.scale, col) : load_scale<false>(p.scale, col);
  if (p.layout == kLayoutTiledI4) {
    const TiledPos pos = tiled_i4_locate(col, group * 32u, p.k, p.scale_f16 ? 2u : 4u);
    return p.scale_f16 ? __half2float(*reinterpret_cast<const __half*>(p.w + pos.scale_offset))
                       : *reinterpret_cast<const float*>(p.w + pos.scale_offset);
  }
  const size_t idx = static_cast<size_t>(col) * (p.k / p.group_size) + group;
  return p.scale_f16 ? load_scale<true>(p.scale, idx) : load_scale<false>(p.scale, idx);
}

__global__ void __launch_bounds__(128) idot_generic_kernel(const IdotParams p) {
  const uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t row = blockIdx.y;
  if (col >= p.n) return;
  const int8_t* xr = p.xq + static_cast<size_t>(row) * p.k;
  if (p.storage == KQ_STORAGE_I8) {
    int acc = 0;
    for (uint32_t kk = 0; kk < p.k; ++kk) acc += static_cast<int>(xr[kk]) * weight_q(p, col, kk);
    const float combined = __fmul_rn(p.xs[row], weight_scale(p, col, 0));
    p.out[static_cast<size_t>(row) * p.n + col] = fmaf(__int2float_rn(acc), combined, p.bias[col]);
    return;
  }
  const uint32_t gsz = p.layout == kLayoutTiledI4 ? 32u : p.group_size;
  float accf = 0.0f;
  for (uint32_t g = 0; g * gsz < p.k; ++g) {
    int acci = 0;
    for (uint32_t kk = g * gsz; kk < (g + 1) * gsz; ++kk) acci += static_cast<int>(xr[kk]) * weight_q(p, col, kk);
    accf = fmaf(__int2float_rn(acci), weight_scale(p, col, g), accf);
  }
  p.out[static_cast<size_t>(row) * p.n + col] = fmaf(accf, p.xs[row], p.bias[col]);
}

// ---- tensor-core integer-dot for the tiled layouts, at most 8 activation rows ---------------
__device__ __forceinline__ void imma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

struct IdotTiledParams {
  const uint8_t* w;
  const void* scale;  // int8: per-channel scales
  int scale_f16;
  uint32_t n, k;
  const int8_t* xq;      // [m, k]
  const float* xs;       // [m]
  const int* row_sum;    // [m]
  const int* group_sum;  // [m, k / 32]
  const float* bias;
  float* out;
  uint32_t m;            // <= 8
};

constexpr int kIdotWarps = 2;
constexpr int kIdotDepth = 4;  // chunks a warp keeps in flight

// int8 weights: chunk (R, J) = 16 rows x 32 k, lane 4g+t holds (a0, a1, a2, a3) of the MMA
// verbatim (bytes q + 128).  One MMA per 512 bytes of weights; the whole K range accumulates
// in int32 (|sum| <= k * 255 * 127, so k <= 65536 is the gate of this kernel).
__global__ void __launch_bounds__(kIdotWarps * 32) idot_w8a8_tiled_kernel(const IdotTiledParams p) {
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t rb = blockIdx.x * kIdotWarps + warp;
  if (rb * 16u >= p.n) return;
  const uint32_t chunks = p.k / 32;
  const uint8_t* src = p.w + static_cast<size_t>(rb) * chunks * 512u + lane * 16;
  // B operand: column g of the MMA is activation row g; k-slots 4t..4t+3 and 16+4t..16+4t+3
  const bool col_live = g < p.m;
  const int8_t* xrow = p.xq + static_cast<size_t>(col_live ? g : 0) * p.k + 4 * t;
  int c[4] = {0, 0, 0, 0};
  // independent loads and one accumulator chain: unrolled, the compiler keeps 8 chunks in flight
#pragma unroll 8
  for (uint32_t j = 0; j < chunks; ++j) {
    const uint4 a = ldg_stream(src + static_cast<size_t>(j) * 512u);
    uint32_t b0 = 0, b1 = 0;
    if (col_live) {
      b0 = __ldg(reinterpret_cast<const uint32_t*>(xrow + j * 32));
      b1 = __ldg(reinterpret_cast<const uint32_t*>(xrow + j * 32 + 16));
    }
    imma_u8s8(c, a.x, a.y, a.z, a.w, b0, b1);
  }
  // c0: (row g, col 2t)  c1: (row g, col 2t+1)  c2: (row g+8, col 2t)  c3: (row g+8, col 2t+1)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t mm = 2 * t + (i & 1), row = rb * 16u + g + ((i >> 1) ? 8u : 0u);
    if (mm >= p.m) continue;
    const int acc = c[i] - 128 * p.row_sum[mm];
    const float ws = p.scale_f16 ? load_scale<true>(p.scale, row) : load_scale<false>(p.scale, row);
    p.out[static_cast<size_t>(mm) * p.n + row] = fmaf(__int2float_rn(acc), __fmul_rn(p.xs[mm], ws), p.bias[row]);
  }
}

// int4 weights (group 32): per group one MMA on (w & 0x0F0F0F0F) [even elements] and
// ((w >> 4) & 0x0F0F0F0F) [odd elements]; the activations are permuted to match with two
// byte permutes; the per-group integer sum is flushed with one fma, groups ascending.
template <bool kScaleF16>
__global__ void __launch_bounds__(kIdotWarps * 32) idot_w4a8_tiled_kernel(const IdotTiledParams p) {
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t rb = blockIdx.x * kIdotWarps + warp;
  if (rb * 16u >= p.n) return;
  const uint32_t chunks = p.k / 64, groups = p.k / 32;
  const uint8_t* src = p.w + static_cast<size_t>(rb) * chunks * kCB;
  const bool col_live = g < p.m;
  const int8_t* xrow = p.xq + static_cast<size_t>(col_live ? g : 0) * p.k + 8 * t;
  const uint32_t m0 = 2 * t, m1 = 2 * t + 1;
  const int* gs0 = p.group_sum + static_cast<size_t>(m0 < p.m ? m0 : 0) * groups;
  const int* gs1 = p.group_sum + static_cast<size_t>(m1 < p.m ? m1 : 0) * groups;
  float accf[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // weights and scales run kIdotDepth chunks ahead of the MMAs, in registers
  using ScaleRegs = typename std::conditional<kScaleF16, uint2, uint4>::type;
  uint4 ring_w[kIdotDepth];
  ScaleRegs ring_s[kIdotDepth];
  auto fetch = [&](int d, uint32_t j) {
    const uint8_t* chunk = src + static_cast<size_t>(j) * kCB;
    ring_w[d] = ldg_stream(chunk + lane * 16);
    if constexpr (kScaleF16) ring_s[d] = __ldg(reinterpret_cast<const uint2*>(chunk + kChunkWeightBytes + g * 8));
    else ring_s[d] = __ldg(reinterpret_cast<const uint4*>(chunk + kChunkWeightBytes + g * 16));
  };
#pragma unroll
  for (int d = 0; d < kIdotDepth; ++d) {
    ring_w[d] = make_uint4(0, 0, 0, 0);
    if constexpr (kScaleF16) ring_s[d] = make_uint2(0, 0);
    else ring_s[d] = make_uint4(0, 0, 0, 0);
    if (static_cast<uint32_t>(d) < chunks) fetch(d, d);
  }
  for (uint32_t j0 = 0; j0 < chunks; j0 += kIdotDepth) {
#pragma unroll
  for (int d = 0; d < kIdotDepth; ++d) {
    const uint32_t j = j0 + d;
    if (j >= chunks) break;
    const uint4 wq = ring_w[d];
    float sc[4];  // row g grp 0 | row g+8 grp 0 | row g grp 1 | row g+8 grp 1
    if constexpr (kScaleF16) {
      const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&ring_s[d].x));
      const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&ring_s[d].y));
      sc[0] = lo.x; sc[1] = lo.y; sc[2] = hi.x; sc[3] = hi.y;
    } else {
      sc[0] = __uint_as_float(ring_s[d].x); sc[1] = __uint_as_float(ring_s[d].y);
      sc[2] = __uint_as_float(ring_s[d].z); sc[3] = __uint_as_float(ring_s[d].w);
    }
    if (j + kIdotDepth < chunks) fetch(d, j + kIdotDepth);
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      const uint32_t group = 2 * j + jj;
      const uint32_t wa = jj ? wq.z : wq.x, wb = jj ? wq.w : wq.y;  // rows g, g + 8
      uint32_t b0 = 0, b1 = 0;
      if (col_live) {
        const uint2 xv = __ldg(reinterpret_cast<const uint2*>(xrow + group * 32));  // elements 8t .. 8t+7
        b0 = __byte_perm(xv.x, xv.y, 0x6420);  // even elements
        b1 = __byte_perm(xv.x, xv.y, 0x7531);  // odd elements
      }
      int c[4] = {0, 0, 0, 0};
      imma_u8s8(c, wa & 0x0F0F0F0Fu, wb & 0x0F0F0F0Fu, (wa >> 4) & 0x0F0F0F0Fu, (wb >> 4) & 0x0F0F0F0Fu, b0, b1);
      const int s0 = 8 * __ldg(gs0 + group), s1 = 8 * __ldg(gs1 + group);
      const float sa = sc[2 * jj], sb = sc[2 * jj + 1];
      accf[0] = fmaf(__int2float_rn(c[0] - s0), sa, accf[0]);
      accf[1] = fmaf(__int2float_rn(c[1] - s1), sa, accf[1]);
      accf[2] = fmaf(__int2float_rn(c[2] - s0), sb, accf[2]);
      accf[3] = fmaf(__int2float_rn(c[3] - s1), sb, accf[3]);
    }
  }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t mm = 2 * t + (i & 1), row = rb * 16u + g + ((i >> 1) ? 8u : 0u);
    if (mm >= p.m) continue;
    p.out[static_cast<size_t>(mm) * p.n + row] = fmaf(accf[i], p.xs[mm], p.bias[row]);
  }
}

}  // namespace

cudaError_t launch_quantize_rows(cudaStream_t stream, const float* x, uint32_t rows, uint32_t dim, int8_t* q,
                                 float* scale, int* row_sum, int* group_sum) {
  if (rows == 0) return cudaSuccess;
  quantize_rows_kernel<<<std::min<uint32_t>(rows, 65535u), 256, 0, stream>>>(x, rows, dim, q, scale, row_sum, group_sum);
  return cudaGetLastError();
}

cudaError_t launch_xq_sums(cudaStream_t stream, const int8_t* q, uint32_t rows, uint32_t dim, int* row_sum,
                           int* group_sum) {
  if (rows == 0) return cudaSuccess;
  xq_sums_kernel<<<rows, 256, 0, stream>>>(q, rows, dim, row_sum, group_sum);
  return cudaGetLastError();
}

// xq / xs as written by launch_quantize_rows; row_sum / group_sum may be null (then only the
// generic kernel is used).  Returns through *launches how many kernels were launched.
cudaError_t launch_linear_idot(cudaStream_t stream, const Weight& w, const int8_t* xq, const float* xs,
                               const int* row_sum, const int* group_sum, const float* bias, float* out,
                               uint32_t m, int* launches) {
  if (m == 0 || w.n == 0) return cudaSuccess;
  const bool tiled8 = w.layout == kLayoutTiledI8 && row_sum != nullptr && w.k <= 65536u;
  const bool tiled4 = w.layout == kLayoutTiledI4 && group_sum != nullptr;
  if (tiled8 || tiled4) {
    for (uint32_t m0 = 0; m0 < m; m0 += 8) {
      IdotTiledParams p = {};
      p.w = static_cast<const uint8_t*>(w.data);
      p.scale = w.scale;
      p.scale_f16 = w.scale_dtype == KQ_F16;
      p.n = w.n;
      p.k = w.k;
      p.xq = xq + static_cast<size_t>(m0) * w.k;
      p.xs = xs + m0;
      p.row_sum = row_sum ? row_sum + m0 : nullptr;
      p.group_sum = group_sum ? group_sum + static_cast<size_t>(m0) * (w.k / 32) : nullptr;
      p.bias = bias;
      p.out = out + static_cast<size_t>(m0) * w.n;
      p.m = std::min<uint32_t>(8u, m - m0);
      const uint32_t grid = (w.n / 16 + kIdotWarps - 1) / kIdotWarps;
      if (tiled8) idot_w8a8_tiled_kernel<<<grid, kIdotWarps * 32, 0, stream>>>(p);
      else if (p.scale_f16) idot_w4a8_tiled_kernel<true><<<grid, kIdotWarps * 32, 0, stream>>>(p);
      else idot_w4a8_tiled_kernel<false><<<grid, kIdotWarps * 32, 0, stream>>>(p);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      if (launches) *launches += 1;
    }
    return cudaSuccess;
  }
  IdotParams p = {};
  p.w = static_cast<const uint8_t*>(w.data);
  p.scale = w.scale;
  p.layout = w.layout;
  p.storage = w.storage;
  p.scale_f16 = w.scale_dtype == KQ_F16;
  p.n = w.n;
  p.k = w.k;
  p.group_size = w.group_size;
  p.xq = xq;
  p.xs = xs;
  p.bias = bias;
  p.out = out;
  p.m = m;
  for (uint32_t m0 = 0; m0 < m; m0 += 65535u) {
    IdotParams q = p;
    q.xq = xq + static_cast<size_t>(m0) * w.k;
    q.xs = xs + m0;
    q.out = out + static_cast<size_t>(m0) * w.n;
    q.m = std::min<uint32_t>(65535u, m - m0);
    idot_generic_kernel<<<dim3((w.n + 127) / 128, q.m), 128, 0, stream>>>(q);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
  }
  return cudaSuccess;
}

}  // namespace kq
