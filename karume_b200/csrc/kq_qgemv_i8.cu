// qgemv_i8 — decode kernel for per-channel int8 weights in the tiled layout (kq_common.cuh),
// 1 <= m <= 16.  Replaces the reference's small-M linear variant with in-kernel int8
// dequant (pipeline key linear:v2:f32:reg16x16r1x4w4:wi8 —
// packages/runtime/src/kernels/weight-storage.ts:191-209 inside gemm.ts:1187-1237).
//
// Same construction as qgemv_i4_kernel (see that file): the stored bytes (q + 128) reach
// mma.sync.m16n8k16 as binary16 subnormals b * 2^-24 after one mask per pair, the
// activations are the B operand staged once per CTA (hi / lo binary16 columns for f32 and
// bf16 input), weights stream through a register ring, K can be split over a cluster and
// is reduced over distributed shared memory in rank order.  Differences: the scale is per
// output channel, so the MMAs of a row simply chain into one f32 accumulator over the
// whole K range and the scale is applied once at the end:
//     y[n] = s[n] * ( sum_k b[n,k] x[k]  -  128 sum_k x[k] ) + bias[n].
// This is the factored form; the bit-exact per-element dequant (one f32 multiply,
// kq::dequant_i8) is what kq_weight_dequant and the generic kernel use.
// Activation domain: any value.  Because the MMAs of a row chain over the whole K range, the
// power-of-two pre-scale of the activations (kq_gemv_core.cuh: pow2_prescale) is chosen per
// activation ROW, from the largest magnitude inside the CTA's own k range, in a short pass
// before the first slab is staged; its inverse multiplies the CTA's partial sum once, in f32.
#include <algorithm>
#include <type_traits>

#include "kq_gemv_core.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kWarps8 = 4;
constexpr int kDepth8 = 4;
constexpr int kMaxCluster8 = 8;
constexpr uint32_t kCB8 = 512;

struct Gemv8Params {
  const uint8_t* w;
  const void* scale;
  const float* bias;
  float* out;
  const void* x;
  uint32_t m, n, k;
  uint32_t chunks_per_split, splits, slab_chunks;
};

__device__ __forceinline__ uint4 ldg_stream_v4_8(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t cluster_map_shared8(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ float ld_cluster_f32_8(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync_all8() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Stages 32-k chunks [chunk0, chunk0 + chunks) of x.
//   xs   : [local chunk][active columns][64 B]; inside a column block, 16 B per t = 0..3:
//          x[4t], x[4t+2], x[4t+1], x[4t+3] of the first 16 k, then the same of the second 16 k
//   corr : [local chunk][kCorrStride] f32 = sum of the chunk's 32 activations as staged
//   row_scale : [m] the 2^e every value of an activation row is multiplied by before the split
template <typename XT, bool kHasLo, int kCorrStride>
__device__ __forceinline__ void stage_x8(const XT* __restrict__ x, uint32_t m, uint32_t k, uint32_t chunk0,
                                         uint32_t chunks, uint8_t* xs, uint32_t xs_stride, float* corr,
                                         const float* row_scale) {
  const uint32_t items = chunks * m * 4;
  const uint32_t items_padded = (items + 31u) & ~31u;
  for (uint32_t item = threadIdx.x; item < items_padded; item += blockDim.x) {
    const bool valid = item < items;
    const uint32_t t = item & 3u;
    const uint32_t rest = item >> 2;
    const uint32_t row = rest % m;
    const uint32_t lc = rest / m;
    uint4 hi4 = make_uint4(0, 0, 0, 0), lo4 = make_uint4(0, 0, 0, 0);
    float sum = 0.0f;
    if (valid) {
      const XT* src = x + static_cast<size_t>(row) * k + (static_cast<size_t>(chunk0 + lc) << 5) + (t << 2);
      const float scale = row_scale[row];
      float v[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[e] = to_f32(src[e]) * scale;
        v[4 + e] = to_f32(src[16 + e]) * scale;
      }
      __half h[8], l[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        h[e] = __float2half_rn(v[e]);
        const float hf = __half2float(h[e]);
        if constexpr (kHasLo) {
          l[e] = __float2half_rn(v[e] - hf);
          sum += hf + __half2float(l[e]);
        } else {
          sum += hf;
        }
      }
      hi4 = make_uint4(pack_half2(h[0], h[2]), pack_half2(h[1], h[3]), pack_half2(h[4], h[6]), pack_half2(h[5], h[7]));
      if constexpr (kHasLo)
        lo4 = make_uint4(pack_half2(l[0], l[2]), pack_half2(l[1], l[3]), pack_half2(l[4], l[6]), pack_half2(l[5], l[7]));
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (valid) {
      const uint32_t col = kHasLo ? 2 * row : row;
      const uint32_t off = lc * xs_stride + col * 64 + t * 16;
      *reinterpret_cast<uint4*>(xs + off) = hi4;
      if constexpr (kHasLo) *reinterpret_cast<uint4*>(xs + off + 64) = lo4;
      if (t == 0) corr[lc * kCorrStride + row] = sum;
    }
  }
}

template <typename XT, bool kScaleF16, int kCols, int kRB>
__global__ void __launch_bounds__(kWarps8 * 32)
qgemv_i8_kernel(const Gemv8Params p) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr int kTiles = kCols / 8;
  constexpr int kCorrPerTile = kHasLo ? 1 : 2;
  constexpr int kCorrStride = kHasLo ? kCols / 2 : kCols;
  constexpr uint32_t kTileRowsCta = kWarps8 * kRB * 16;
  constexpr uint32_t kMask = 0x00FF00FFu;  // bytes 0 and 2 of a word: b * 2^-24 as binary16

  extern __shared__ __align__(16) uint8_t smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  pdl_launch_dependents();

  const uint32_t tile = blockIdx.x;
  const uint32_t row_block0 = (tile * kWarps8 + warp) * kRB;
  const uint32_t chunks_per_row = p.k / kChunkK8;
  const uint32_t split = blockIdx.y;
  const uint32_t cbeg = min(split * p.chunks_per_split, chunks_per_row);
  const uint32_t cend = min(cbeg + p.chunks_per_split, chunks_per_row);
  const uint32_t nch = cend - cbeg;
  const uint32_t active_cols = kHasLo ? 2 * p.m : p.m;
  const uint32_t xs_stride = active_cols * 64;
  uint8_t* xs = smem;
  float* corr = reinterpret_cast<float*>(smem + p.slab_chunks * xs_stride);

  bool active[kRB];
  const uint8_t* next[kRB];
#pragma unroll
  for (int r = 0; r < kRB; ++r) {
    active[r] = (row_block0 + r) * 16u < p.n;
    next[r] = p.w + (static_cast<size_t>(row_block0 + r) * chunks_per_row + cbeg) * kCB8 + lane * 16;
  }
  uint4 ring[kDepth8][kRB];
#pragma unroll
  for (int d = 0; d < kDepth8; ++d)
#pragma unroll
    for (int r = 0; r < kRB; ++r) {
      ring[d][r] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);  // q = 0
      if (active[r] && static_cast<uint32_t>(d) < nch) ring[d][r] = ldg_stream_v4_8(next[r] + d * kCB8);
    }
#pragma unroll
  for (int r = 0; r < kRB; ++r) next[r] += kDepth8 * kCB8;

  pdl_wait_prior_grid();

  // Per activation row: largest magnitude inside this CTA's k range -> 2^e and 2^-e.
  __shared__ float amax_part[kWarps8][16];
  __shared__ float row_scale[16], row_inv[16];
  {
    const XT* xin = static_cast<const XT*>(p.x);
    const uint32_t k0 = cbeg * kChunkK8, k1 = cend * kChunkK8;
    for (uint32_t row = 0; row < p.m; ++row) {
      float amax = 0.0f;
      for (uint32_t i = k0 + threadIdx.x * 8; i < k1; i += blockDim.x * 8) {
        float v[8];
        load_x8<XT>(xin + static_cast<size_t>(row) * p.k + i, v);
        amax = fmaxf(amax, absmax8(v));
      }
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
      if (lane == 0) amax_part[warp][row] = amax;
    }
    __syncthreads();
    if (threadIdx.x < p.m) {
      float amax = amax_part[0][threadIdx.x];
#pragma unroll
      for (int w = 1; w < kWarps8; ++w) amax = fmaxf(amax, amax_part[w][threadIdx.x]);
      const Pow2 ps = pow2_prescale(amax);
      row_scale[threadIdx.x] = ps.scale;
      row_inv[threadIdx.x] = ps.inv;
    }
    __syncthreads();
  }

  float acc[kRB][kTiles][4];  // MMA accumulators over the whole K range of this CTA
  float csum[kTiles][kCorrPerTile];
#pragma unroll
  for (int r = 0; r < kRB; ++r)
#pragma unroll
    for (int i = 0; i < kTiles; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[r][i][j] = 0.0f;
  uint4 bfrag[kTiles];
  float cterm[kTiles][kCorrPerTile];
  bool load_b[kTiles], load_c[kTiles][kCorrPerTile];
#pragma unroll
  for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
    bfrag[tile_m] = make_uint4(0, 0, 0, 0);
    load_b[tile_m] = tile_m * 8 + g < active_cols;
#pragma unroll
    for (int j = 0; j < kCorrPerTile; ++j) {
      cterm[tile_m][j] = 0.0f;
      csum[tile_m][j] = 0.0f;
      const uint32_t mm = kHasLo ? tile_m * 4 + t : tile_m * 8 + 2 * t + j;
      load_c[tile_m][j] = mm < p.m;
    }
  }
  const uint32_t xs_lane = static_cast<uint32_t>(__cvta_generic_to_shared(xs)) + lane * 16;
  const uint32_t corr_lane = static_cast<uint32_t>(__cvta_generic_to_shared(corr)) + (kHasLo ? t : 2 * t) * 4;
  const XT* x = static_cast<const XT*>(p.x);

  auto process = [&](const int d, uint32_t xs_addr, uint32_t corr_addr, bool refill) {
#pragma unroll
    for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
      lds_v4_if(bfrag[tile_m], xs_addr + tile_m * 512, load_b[tile_m]);
#pragma unroll
      for (int j = 0; j < kCorrPerTile; ++j) {
        lds_f32_if(cterm[tile_m][j], corr_addr + (tile_m * (kHasLo ? 4 : 8) + j) * 4, load_c[tile_m][j]);
        csum[tile_m][j] += cterm[tile_m][j];
      }
    }
#pragma unroll
    for (int r = 0; r < kRB; ++r) {
      const uint4 wq = ring[d][r];
      const uint32_t a0[4] = {wq.x & kMask, wq.y & kMask, (wq.x >> 8) & kMask, (wq.y >> 8) & kMask};
      const uint32_t a1[4] = {wq.z & kMask, wq.w & kMask, (wq.z >> 8) & kMask, (wq.w >> 8) & kMask};
#pragma unroll
      for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
        mma_f16(acc[r][tile_m], a0, bfrag[tile_m].x, bfrag[tile_m].y);
        mma_f16(acc[r][tile_m], a1, bfrag[tile_m].z, bfrag[tile_m].w);
      }
    }
    if (refill) {
#pragma unroll
      for (int r = 0; r < kRB; ++r)
        if (active[r]) ring[d][r] = ldg_stream_v4_8(next[r] + d * kCB8);
    }
  };

  for (uint32_t done = 0; done < nch;) {
    const uint32_t slab_n = min(p.slab_chunks, nch - done);
    if (done != 0) __syncthreads();
    stage_x8<XT, kHasLo, kCorrStride>(x, p.m, p.k, cbeg + done, slab_n, xs, xs_stride, corr, row_scale);
    __syncthreads();
    uint32_t xs_addr = xs_lane, corr_addr = corr_lane;
    uint32_t i = 0;
    for (; i + kDepth8 <= slab_n; i += kDepth8) {
#pragma unroll
      for (int d = 0; d < kDepth8; ++d) {
        process(d, xs_addr, corr_addr, done + i + d + kDepth8 < nch);
        xs_addr += xs_stride;
        corr_addr += kCorrStride * 4;
      }
#pragma unroll
      for (int r = 0; r < kRB; ++r) next[r] += kDepth8 * kCB8;
    }
#pragma unroll
    for (int d = 0; d < kDepth8 - 1; ++d) {
      if (i + d < slab_n) {
        process(d, xs_addr, corr_addr, false);
        xs_addr += xs_stride;
        corr_addr += kCorrStride * 4;
      }
    }
    done += slab_n;
  }

  // ---- epilogue: value(row, mm) = 2^24 * (accumulated b.x) - 128 * sum x ; out = s * value + bias
  float* red = reinterpret_cast<float*>(smem);
  if (p.splits > 1) __syncthreads();
#pragma unroll
  for (int r = 0; r < kRB; ++r) {
    if (!active[r]) continue;
    const uint32_t row_a = (row_block0 + r) * 16u + g;
    const uint32_t tr_a = (warp * kRB + r) * 16u + g;
    float s_a = 0.0f, s_b = 0.0f, bias_a = 0.0f, bias_b = 0.0f;
    if (p.splits == 1) {
      s_a = load_scale<kScaleF16>(p.scale, row_a);
      s_b = load_scale<kScaleF16>(p.scale, row_a + 8);
      bias_a = p.bias[row_a];
      bias_b = p.bias[row_a + 8];
    }
#pragma unroll
    for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
#pragma unroll
      for (int j = 0; j < (kHasLo ? 1 : 2); ++j) {
        const uint32_t mm = kHasLo ? tile_m * 4 + t : tile_m * 8 + 2 * t + j;
        if (mm >= p.m) continue;
        const float ca = kHasLo ? acc[r][tile_m][0] + acc[r][tile_m][1] : acc[r][tile_m][j];
        const float cb = kHasLo ? acc[r][tile_m][2] + acc[r][tile_m][3] : acc[r][tile_m][2 + j];
        const float off = -128.0f * csum[tile_m][kHasLo ? 0 : j];
        const float inv = row_inv[mm];  // undo the row's power-of-two pre-scale (exact)
        const float va = fmaf(ca, kUnscale, off) * inv, vb = fmaf(cb, kUnscale, off) * inv;
        if (p.splits == 1) {
          p.out[static_cast<size_t>(mm) * p.n + row_a] = fmaf(s_a, va, bias_a);
          p.out[static_cast<size_t>(mm) * p.n + row_a + 8] = fmaf(s_b, vb, bias_b);
        } else {
          red[mm * kTileRowsCta + tr_a] = va;
          red[mm * kTileRowsCta + tr_a + 8] = vb;
        }
      }
    }
  }
  if (p.splits == 1) return;
  cluster_sync_all8();
  const uint32_t rows_here = min(kTileRowsCta, p.n - tile * kTileRowsCta);
  const uint32_t total = rows_here * p.m;
  const uint32_t per_rank = (total + p.splits - 1) / p.splits;
  const uint32_t lo = min(split * per_rank, total), hi = min(lo + per_rank, total);
  const uint32_t red_base = static_cast<uint32_t>(__cvta_generic_to_shared(red));
  for (uint32_t idx = lo + threadIdx.x; idx < hi; idx += blockDim.x) {
    const uint32_t mm = idx / rows_here, r = idx - mm * rows_here;
    const uint32_t local = red_base + (mm * kTileRowsCta + r) * 4u;
    float sum = 0.0f;
    for (uint32_t s = 0; s < p.splits; ++s) sum += ld_cluster_f32_8(cluster_map_shared8(local, s));
    const uint32_t row = tile * kTileRowsCta + r;
    p.out[static_cast<size_t>(mm) * p.n + row] = fmaf(load_scale<kScaleF16>(p.scale, row), sum, p.bias[row]);
  }
  cluster_sync_all8();
}

template <typename XT, bool kScaleF16, int kCols, int kRB>
cudaError_t launch_typed8(const LaunchEnv& env, Gemv8Params& p) {
  auto kernel = qgemv_i8_kernel<XT, kScaleF16, kCols, kRB>;
  struct Setup { bool done; uint32_t max_cluster; };
  static PerDevice<Setup> setup_on;
  Setup* setup = setup_on.slot();
  if (setup == nullptr) return cudaErrorInvalidDevice;
  uint32_t& max_cluster = setup->max_cluster;
  if (!setup->done) {
    max_cluster = kMaxCluster8;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return e;
    // few row tiles and a long k: sixteen splits (the largest cluster, by opt-in)
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) max_cluster = 16;
    else (void)cudaGetLastError();
    setup->done = true;
  }
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kTileRowsCta = kWarps8 * kRB * 16;
  const uint32_t tiles = (p.n + kTileRowsCta - 1) / kTileRowsCta;
  const uint32_t chunks_per_row = p.k / kChunkK8;
  const uint32_t want_ctas = static_cast<uint32_t>(env.sm_count) * 4u;
  uint32_t splits = 1;
  // once every SM has a CTA, a split keeps at least twelve 32-k chunks: below that a CTA's fixed
  // cost outweighs its share of the stream
  while (splits < max_cluster && tiles * splits < want_ctas && splits * 2 <= chunks_per_row &&
         (tiles * splits < static_cast<uint32_t>(env.sm_count) || splits * 2 * 12 <= chunks_per_row))
    splits *= 2;
  p.splits = splits;
  p.chunks_per_split = (chunks_per_row + splits - 1) / splits;
  const uint32_t per_chunk = (kHasLo ? 2 * p.m : p.m) * 64 + (kHasLo ? kCols / 2 : kCols) * 4;
  const uint32_t slab_cap = std::max<uint32_t>(kDepth8, (32768u / per_chunk) / kDepth8 * kDepth8);
  p.slab_chunks = std::max<uint32_t>(1u, std::min(p.chunks_per_split, slab_cap));
  const size_t slab_bytes = static_cast<size_t>(p.slab_chunks) * per_chunk;
  const size_t red_bytes = splits > 1 ? static_cast<size_t>(p.m) * kTileRowsCta * sizeof(float) : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, splits, 1);
  cfg.blockDim = dim3(kWarps8 * 32, 1, 1);
  cfg.dynamicSmemBytes = std::max(slab_bytes, red_bytes);
  cfg.stream = env.stream;
  cudaLaunchAttribute attr[2];
  unsigned int na = 0;
  if (env.overlap) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (splits > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = splits;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

template <typename XT>
cudaError_t launch_x8(const LaunchEnv& env, Gemv8Params& p, bool f16s) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  const uint32_t cols = kHasLo ? 2 * p.m : p.m;
  if (cols <= 8) return f16s ? launch_typed8<XT, true, 8, 1>(env, p) : launch_typed8<XT, false, 8, 1>(env, p);
  if (cols <= 16) return f16s ? launch_typed8<XT, true, 16, 2>(env, p) : launch_typed8<XT, false, 16, 2>(env, p);
  if constexpr (kHasLo) {
    return f16s ? launch_typed8<XT, true, 32, 2>(env, p) : launch_typed8<XT, false, 32, 2>(env, p);
  } else {
    return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_qgemv_i8(const LaunchEnv& env, const LinearTarget& target, const void* x, int x_dtype,
                            uint32_t m) {
  const Weight& w = *target.w;
  if (w.layout != kLayoutTiledI8 || m < 1 || m > 16) return cudaErrorInvalidValue;
  Gemv8Params p = {};
  p.w = static_cast<const uint8_t*>(w.data);
  p.scale = w.scale;
  p.bias = target.bias;
  p.out = target.out;
  p.x = x;
  p.m = m;
  p.n = w.n;
  p.k = w.k;
  const bool f16s = w.scale_dtype == KQ_F16;
  switch (x_dtype) {
    case KQ_F32: return launch_x8<float>(env, p, f16s);
    case KQ_F16: return launch_x8<__half>(env, p, f16s);
    case KQ_BF16: return launch_x8<__nv_bfloat16>(env, p, f16s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace kq
