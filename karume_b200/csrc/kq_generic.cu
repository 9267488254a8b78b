// Shape-generic kernels of libkq: the quantized linear for every shape the storage
// contract allows (the counterpart of the reference's scalar / small-tile variants,
// packages/runtime/src/kernels/gemm-geometry.ts:243-267), the f32 expansion of a
// resident weight, and the repack into the tiled int4 layout.
//
// The generic linear keeps the reference's arithmetic form literally: every weight
// is dequantised with one f32 multiply and then enters an FMA with the activation
// (packages/runtime/src/kernels/gemm.ts:642-718 fill, :922-940 MAC), f32 accumulate,
// bias added once after the K reduction (:862-873).  Only the summation tree differs
// (32 lanes stride K, then a shuffle tree), which the stated tolerance covers.
#include "kq_common.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kGenericWarps = 4;
constexpr int kGenericMT = 4;  // activation rows handled per pass

// ---- int4, native layout ---------------------------------------------------------
// One warp per output channel.  k % 16 == 0 always holds for int4 (group size is a
// power of two >= 16 dividing k), so a row starts on an 8-byte boundary and a 32-bit
// word (8 elements) never straddles a scale group.
template <typename XT, bool kScaleF16>
__global__ void __launch_bounds__(kGenericWarps * 32)
linear_generic_i4(const uint32_t* __restrict__ w, const void* __restrict__ scale,
                  const XT* __restrict__ x, const float* __restrict__ bias,
                  float* __restrict__ out, uint32_t m, uint32_t n, uint32_t k, uint32_t gshift) {
  pdl_launch_dependents();
  pdl_wait_prior_grid();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t col = blockIdx.x * kGenericWarps + (threadIdx.x >> 5);
  const uint32_t m0 = blockIdx.y * kGenericMT;
  if (col >= n) return;
  const uint32_t words = k >> 3;
  const uint32_t groups = k >> gshift;
  const uint32_t* wrow = w + static_cast<size_t>(col) * words;
  float acc[kGenericMT];
#pragma unroll
  for (int r = 0; r < kGenericMT; ++r) acc[r] = 0.0f;
  for (uint32_t wi = lane; wi < words; wi += 32) {
    const uint32_t word = wrow[wi];
    const uint32_t kbase = wi << 3;
    const float s = load_scale<kScaleF16>(scale, static_cast<size_t>(col) * groups + (kbase >> gshift));
    float wv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) wv[e] = dequant_i4((word >> (4 * e)) & 0xFu, s);
#pragma unroll
    for (int r = 0; r < kGenericMT; ++r) {
      if (m0 + r < m) {
        const XT* xr = x + static_cast<size_t>(m0 + r) * k + kbase;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[r] = fmaf(to_f32(xr[e]), wv[e], acc[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kGenericMT; ++r) {
    const float total = warp_sum(acc[r]);
    if (lane == 0 && m0 + r < m) out[static_cast<size_t>(m0 + r) * n + col] = total + bias[col];
  }
}

// ---- int8, native layout -----------------------------------------------------------
// k is arbitrary (the reference tests k = 7 and k = 20), so weights are read byte-wise
// from the flat index col*k + i, exactly the "word = i/4, lane = i%4" rule of
// docs/ir-v1.md:170-176 without assuming any row alignment.
template <typename XT, bool kScaleF16>
__global__ void __launch_bounds__(kGenericWarps * 32)
linear_generic_i8(const int8_t* __restrict__ w, const void* __restrict__ scale,
                  const XT* __restrict__ x, const float* __restrict__ bias,
                  float* __restrict__ out, uint32_t m, uint32_t n, uint32_t k) {
  pdl_launch_dependents();
  pdl_wait_prior_grid();
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t col = blockIdx.x * kGenericWarps + (threadIdx.x >> 5);
  const uint32_t m0 = blockIdx.y * kGenericMT;
  if (col >= n) return;
  const int8_t* wrow = w + static_cast<size_t>(col) * k;
  const float s = load_scale<kScaleF16>(scale, col);
  float acc[kGenericMT];
#pragma unroll
  for (int r = 0; r < kGenericMT; ++r) acc[r] = 0.0f;
  if ((k & 15u) == 0) {
    // rows are 16-byte aligned: 16 weights per 128-bit load
    const uint4* wrow16 = reinterpret_cast<const uint4*>(wrow);
    for (uint32_t vi = lane; vi < (k >> 4); vi += 32) {
      const uint4 v = wrow16[vi];
      const uint32_t parts[4] = {v.x, v.y, v.z, v.w};
      float wv[16];
#pragma unroll
      for (int e = 0; e < 16; ++e)
        wv[e] = dequant_i8(static_cast<int>(static_cast<int8_t>((parts[e >> 2] >> (8 * (e & 3))) & 0xFFu)), s);
#pragma unroll
      for (int r = 0; r < kGenericMT; ++r) {
        if (m0 + r < m) {
          const XT* xr = x + static_cast<size_t>(m0 + r) * k + (vi << 4);
#pragma unroll
          for (int e = 0; e < 16; ++e) acc[r] = fmaf(to_f32(xr[e]), wv[e], acc[r]);
        }
      }
    }
  } else {
    for (uint32_t i = lane; i < k; i += 32) {
      const float wv = dequant_i8(static_cast<int>(wrow[i]), s);
#pragma unroll
      for (int r = 0; r < kGenericMT; ++r)
        if (m0 + r < m) acc[r] = fmaf(to_f32(x[static_cast<size_t>(m0 + r) * k + i]), wv, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < kGenericMT; ++r) {
    const float total = warp_sum(acc[r]);
    if (lane == 0 && m0 + r < m) out[static_cast<size_t>(m0 + r) * n + col] = total + bias[col];
  }
}

// ---- f32 expansion -----------------------------------------------------------------
template <bool kScaleF16>
__global__ void dequant_native_i4(const uint8_t* __restrict__ w, const void* __restrict__ scale,
                                  float* __restrict__ out, uint32_t n, uint32_t k, uint32_t gshift) {
  const size_t total = static_cast<size_t>(n) * k;
  const uint32_t groups = k >> gshift;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint32_t row = static_cast<uint32_t>(i / k), kk = static_cast<uint32_t>(i % k);
    const uint8_t byte = w[i >> 1];
    const uint32_t u = (i & 1) ? (byte >> 4) : (byte & 0x0Fu);
    out[i] = dequant_i4(u, load_scale<kScaleF16>(scale, static_cast<size_t>(row) * groups + (kk >> gshift)));
  }
}

template <bool kScaleF16>
__global__ void dequant_tiled_i4(const uint8_t* __restrict__ tiled, float* __restrict__ out,
                                 uint32_t n, uint32_t k) {
  const size_t total = static_cast<size_t>(n) * k;
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint32_t row = static_cast<uint32_t>(i / k), kk = static_cast<uint32_t>(i % k);
    const TiledPos pos = tiled_i4_locate(row, kk, k, kScaleBytes);
    const uint32_t word = *reinterpret_cast<const uint32_t*>(tiled + pos.word_offset);
    const float s = load_scale<kScaleF16>(tiled + pos.scale_offset, 0);
    out[i] = dequant_i4((word >> (4 * pos.nibble)) & 0xFu, s);
  }
}

template <bool kScaleF16>
__global__ void dequant_native_i8(const int8_t* __restrict__ w, const void* __restrict__ scale,
                                  float* __restrict__ out, uint32_t n, uint32_t k) {
  const size_t total = static_cast<size_t>(n) * k;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    out[i] = dequant_i8(static_cast<int>(w[i]), load_scale<kScaleF16>(scale, i / k));
  }
}

template <bool kScaleF16>
__global__ void dequant_tiled_i8(const uint8_t* __restrict__ tiled, const void* __restrict__ scale,
                                 float* __restrict__ out, uint32_t n, uint32_t k) {
  const size_t total = static_cast<size_t>(n) * k;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint32_t row = static_cast<uint32_t>(i / k), kk = static_cast<uint32_t>(i % k);
    const int q = static_cast<int>(tiled[tiled_i8_locate(row, kk, k)]) - 128;  // stored with the sign bit flipped
    out[i] = dequant_i8(q, load_scale<kScaleF16>(scale, row));
  }
}

// ---- embedding gather -----------------------------------------------------------------
// out[row, col] = dequant(weight[index[row], col]) — the reference's embedding kernel with a
// packed weight (packages/runtime/src/kernels/embedding.ts:70-117): same dequant rule as the
// linear (one f32 multiply), group scale looked up per element for int4, and an index outside
// [0, vocab) poisons its output elements with a quiet NaN instead of returning another row.
struct EmbeddingParams {
  const uint8_t* w;
  const void* scale;
  int layout, storage, scale_f16;
  uint32_t vocab, hidden, gshift;
  const int* index;
  float* out;
  uint64_t total;  // rows * hidden
};

__global__ void __launch_bounds__(256) embedding_kernel(const EmbeddingParams p) {
  for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < p.total;
       i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint32_t row = static_cast<uint32_t>(i / p.hidden), col = static_cast<uint32_t>(i % p.hidden);
    const int pick = p.index[row];
    float v;
    if (pick < 0 || static_cast<uint32_t>(pick) >= p.vocab) {
      v = __int_as_float(0x7fc00000);
    } else if (p.storage == KQ_STORAGE_I4) {
      if (p.layout == kLayoutTiledI4) {
        const TiledPos pos = tiled_i4_locate(static_cast<uint32_t>(pick), col, p.hidden, p.scale_f16 ? 2u : 4u);
        const uint32_t word = *reinterpret_cast<const uint32_t*>(p.w + pos.word_offset);
        const float s = p.scale_f16 ? load_scale<true>(p.w + pos.scale_offset, 0) : load_scale<false>(p.w + pos.scale_offset, 0);
        v = dequant_i4((word >> (4 * pos.nibble)) & 0xFu, s);
      } else {
        const uint64_t flat = static_cast<uint64_t>(pick) * p.hidden + col;
        const uint8_t byte = p.w[flat >> 1];
        const uint32_t u = (flat & 1) ? (byte >> 4) : (byte & 0x0Fu);
        const size_t si = static_cast<size_t>(pick) * (p.hidden >> p.gshift) + (col >> p.gshift);
        v = dequant_i4(u, p.scale_f16 ? load_scale<true>(p.scale, si) : load_scale<false>(p.scale, si));
      }
    } else {
      const int q = p.layout == kLayoutTiledI8
                        ? static_cast<int>(p.w[tiled_i8_locate(static_cast<uint32_t>(pick), col, p.hidden)]) - 128
                        : static_cast<int>(reinterpret_cast<const int8_t*>(p.w)[static_cast<uint64_t>(pick) * p.hidden + col]);
      v = dequant_i8(q, p.scale_f16 ? load_scale<true>(p.scale, pick) : load_scale<false>(p.scale, pick));
    }
    p.out[i] = v;
  }
}

// One thread per 32-bit word of the destination.
__global__ void repack_i8_tiled(const uint8_t* __restrict__ payload, uint32_t n, uint32_t k,
                                uint8_t* __restrict__ tiled) {
  const uint32_t chunks_per_block = k / kChunkK8;
  const size_t total = static_cast<size_t>(n / kTileRows) * chunks_per_block * 128;
  for (size_t it = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; it < total;
       it += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t chunk = it >> 7;
    const uint32_t item = static_cast<uint32_t>(it & 127u);
    const uint32_t R = static_cast<uint32_t>(chunk / chunks_per_block), J = static_cast<uint32_t>(chunk % chunks_per_block);
    const uint32_t lane = item >> 2, word = item & 3u, g = lane >> 2, t = lane & 3u;
    const uint32_t row = R * kTileRows + g + ((word & 1u) ? 8u : 0u);
    const uint32_t kk = J * kChunkK8 + (word >> 1) * 16u + t * 4u;
    const uint32_t v = *reinterpret_cast<const uint32_t*>(payload + static_cast<size_t>(row) * k + kk);
    *reinterpret_cast<uint32_t*>(tiled + chunk * 512u + lane * 16u + word * 4u) = v ^ 0x80808080u;
  }
}

// ---- repack into the tiled layout ----------------------------------------------------
// One thread per 32-bit word of the destination (weights first, then scales).
__global__ void repack_i4_tiled(const uint8_t* __restrict__ payload, const uint8_t* __restrict__ scale,
                                uint32_t scale_bytes_per_elem, uint32_t n, uint32_t k,
                                uint8_t* __restrict__ tiled) {
  const uint32_t chunks_per_block = k / kChunkK;
  const size_t chunks = static_cast<size_t>(n / kTileRows) * chunks_per_block;
  const uint32_t cb = chunk_bytes(scale_bytes_per_elem);
  const uint32_t scale_entries = 32;  // 8 g x 4 values
  const uint32_t items_per_chunk = 128 + scale_entries;
  const size_t total = chunks * items_per_chunk;
  const uint32_t groups = k >> 5;
  for (size_t it = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; it < total;
       it += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t chunk = it / items_per_chunk;
    const uint32_t item = static_cast<uint32_t>(it % items_per_chunk);
    const uint32_t R = static_cast<uint32_t>(chunk / chunks_per_block);
    const uint32_t J = static_cast<uint32_t>(chunk % chunks_per_block);
    uint8_t* dst = tiled + chunk * cb;
    if (item < 128) {
      const uint32_t lane = item >> 2, word = item & 3u;
      const uint32_t g = lane >> 2, t = lane & 3u;
      const uint32_t row = R * kTileRows + g + ((word & 1u) ? 8u : 0u);
      const uint32_t group = 2 * J + (word >> 1);
      const size_t src = static_cast<size_t>(row) * (k >> 1) + group * 16u + t * 4u;
      *reinterpret_cast<uint32_t*>(dst + lane * 16u + word * 4u) =
          *reinterpret_cast<const uint32_t*>(payload + src);
    } else {
      const uint32_t entry = item - 128;  // g*4 + jj*2 + upper
      const uint32_t g = entry >> 2, jj = (entry >> 1) & 1u, upper = entry & 1u;
      const uint32_t row = R * kTileRows + g + upper * 8u;
      const size_t src = (static_cast<size_t>(row) * groups + 2 * J + jj) * scale_bytes_per_elem;
      uint8_t* d = dst + kChunkWeightBytes + entry * scale_bytes_per_elem;
      if (scale_bytes_per_elem == 2) {
        *reinterpret_cast<uint16_t*>(d) = *reinterpret_cast<const uint16_t*>(scale + src);
      } else {
        *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(scale + src);
      }
    }
  }
}

uint32_t log2_exact(uint32_t v) {
  uint32_t s = 0;
  while ((1u << s) < v) ++s;
  return s;
}

template <typename XT>
cudaError_t launch_generic_typed(const LaunchEnv& env, const Weight& w, const XT* x,
                                 const float* bias, float* out, uint32_t m) {
  if (m == 0 || w.n == 0) return cudaSuccess;
  const dim3 grid((w.n + kGenericWarps - 1) / kGenericWarps, (m + kGenericMT - 1) / kGenericMT);
  const dim3 block(kGenericWarps * 32);
  const bool f16s = w.scale_dtype == KQ_F16;
  if (w.storage == KQ_STORAGE_I4) {
    const uint32_t gshift = log2_exact(w.group_size);
    if (f16s)
      linear_generic_i4<XT, true><<<grid, block, 0, env.stream>>>(
          static_cast<const uint32_t*>(w.data), w.scale, x, bias, out, m, w.n, w.k, gshift);
    else
      linear_generic_i4<XT, false><<<grid, block, 0, env.stream>>>(
          static_cast<const uint32_t*>(w.data), w.scale, x, bias, out, m, w.n, w.k, gshift);
  } else {
    if (f16s)
      linear_generic_i8<XT, true><<<grid, block, 0, env.stream>>>(
          static_cast<const int8_t*>(w.data), w.scale, x, bias, out, m, w.n, w.k);
    else
      linear_generic_i8<XT, false><<<grid, block, 0, env.stream>>>(
          static_cast<const int8_t*>(w.data), w.scale, x, bias, out, m, w.n, w.k);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_linear_generic(const LaunchEnv& env, const Weight& w, const void* x, int x_dtype,
                                  const float* bias, float* out, uint32_t m) {
  if (w.layout != kLayoutNative) return cudaErrorInvalidValue;
  switch (x_dtype) {
    case KQ_F32: return launch_generic_typed(env, w, static_cast<const float*>(x), bias, out, m);
    case KQ_F16: return launch_generic_typed(env, w, static_cast<const __half*>(x), bias, out, m);
    case KQ_BF16: return launch_generic_typed(env, w, static_cast<const __nv_bfloat16*>(x), bias, out, m);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_dequant(const LaunchEnv& env, const Weight& w, float* out) {
  const size_t total = static_cast<size_t>(w.n) * w.k;
  if (total == 0) return cudaSuccess;
  const int block = 256;
  const int grid = static_cast<int>(std::min<size_t>((total + block - 1) / block, static_cast<size_t>(env.sm_count) * 16));
  const bool f16s = w.scale_dtype == KQ_F16;
  if (w.storage == KQ_STORAGE_I4 && w.layout == kLayoutTiledI4) {
    if (f16s) dequant_tiled_i4<true><<<grid, block, 0, env.stream>>>(static_cast<const uint8_t*>(w.data), out, w.n, w.k);
    else dequant_tiled_i4<false><<<grid, block, 0, env.stream>>>(static_cast<const uint8_t*>(w.data), out, w.n, w.k);
  } else if (w.storage == KQ_STORAGE_I8 && w.layout == kLayoutTiledI8) {
    if (f16s) dequant_tiled_i8<true><<<grid, block, 0, env.stream>>>(static_cast<const uint8_t*>(w.data), w.scale, out, w.n, w.k);
    else dequant_tiled_i8<false><<<grid, block, 0, env.stream>>>(static_cast<const uint8_t*>(w.data), w.scale, out, w.n, w.k);
  } else if (w.storage == KQ_STORAGE_I4) {
    const uint32_t gshift = log2_exact(w.group_size);
    if (f16s) dequant_native_i4<true><<<grid, block, 0, env.stream>>>(static_cast<const uint8_t*>(w.data), w.scale, out, w.n, w.k, gshift);
    else dequant_native_i4<false><<<grid, block, 0, env.stream>>>(static_cast<const uint8_t*>(w.data), w.scale, out, w.n, w.k, gshift);
  } else {
    if (f16s) dequant_native_i8<true><<<grid, block, 0, env.stream>>>(static_cast<const int8_t*>(w.data), w.scale, out, w.n, w.k);
    else dequant_native_i8<false><<<grid, block, 0, env.stream>>>(static_cast<const int8_t*>(w.data), w.scale, out, w.n, w.k);
  }
  return cudaGetLastError();
}

cudaError_t launch_embedding(const LaunchEnv& env, const Weight& w, const int* index, uint32_t rows, float* out) {
  const uint64_t total = static_cast<uint64_t>(rows) * w.k;
  if (total == 0) return cudaSuccess;
  EmbeddingParams p = {};
  p.w = static_cast<const uint8_t*>(w.data);
  p.scale = w.scale;
  p.layout = w.layout;
  p.storage = w.storage;
  p.scale_f16 = w.scale_dtype == KQ_F16;
  p.vocab = w.n;
  p.hidden = w.k;
  p.gshift = w.storage == KQ_STORAGE_I4 ? log2_exact(w.group_size) : 0;
  p.index = index;
  p.out = out;
  p.total = total;
  const int block = 256;
  const int grid = static_cast<int>(std::min<uint64_t>((total + block - 1) / block, static_cast<uint64_t>(env.sm_count) * 16));
  embedding_kernel<<<grid, block, 0, env.stream>>>(p);
  return cudaGetLastError();
}

bool tiled_i4_eligible(int storage, uint32_t n, uint32_t k, uint32_t group_size) {
  return storage == KQ_STORAGE_I4 && group_size == 32 && n > 0 && k > 0 && n % kTileRows == 0 &&
         k % kChunkK == 0;
}

bool tiled_i8_eligible(int storage, uint32_t n, uint32_t k) {
  return storage == KQ_STORAGE_I8 && n > 0 && k > 0 && n % kTileRows == 0 && k % kChunkK8 == 0;
}

cudaError_t launch_repack_i8(cudaStream_t stream, const uint8_t* payload, uint32_t n, uint32_t k, uint8_t* tiled) {
  const size_t total = static_cast<size_t>(n / kTileRows) * (k / kChunkK8) * 128;
  const int block = 256;
  const int grid = static_cast<int>(std::min<size_t>((total + block - 1) / block, 148u * 32u));
  repack_i8_tiled<<<grid, block, 0, stream>>>(payload, n, k, tiled);
  return cudaGetLastError();
}

cudaError_t launch_repack_i4(cudaStream_t stream, const uint8_t* payload, const void* scale,
                             int scale_dtype, uint32_t n, uint32_t k, uint8_t* tiled) {
  const uint32_t sb = scale_dtype == KQ_F16 ? 2u : 4u;
  const size_t total = static_cast<size_t>(n / kTileRows) * (k / kChunkK) * 160;
  const int block = 256;
  const int grid = static_cast<int>(std::min<size_t>((total + block - 1) / block, 148u * 32u));
  repack_i4_tiled<<<grid, block, 0, stream>>>(payload, static_cast<const uint8_t*>(scale), sb, n, k, tiled);
  return cudaGetLastError();
}

}  // namespace kq
