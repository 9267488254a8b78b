// qgemv_i4 — the decode-path kernel of libkq: y[m, n] = x[m, k] . W[n, k]^T + b for
// 1 <= m <= 16 with W in the tiled int4 / group-32 layout (kq_common.cuh).
//
// Replaces the reference's small-M linear variant with in-kernel int4 dequant
// (pipeline key linear:v2:f32:reg16x16r1x4w4:wi4g32 — packages/runtime/src/kernels/
// gemm.ts:1187-1237 with geometry packages/runtime/src/kernels/gemm-geometry.ts:243).
//
// Why it looks the way it does.  The kernel has to be HBM-bound: 0.5625 bytes per
// weight at ~6.5 TB/s is ~11.5e12 weights/s, which leaves about three issue slots per
// weight on 148 SMs — not enough for "unpack, convert, scale, FMA" per weight on the
// FP32 pipe, and nothing at all for m > 1.  So:
//   * weights stream through a per-warp cp.async ring (128-bit per lane, 8 stages,
//     no register staging, no block-wide barrier in the steady state);
//   * a nibble is never converted: `word & 0x000F000F` IS a pair of binary16
//     subnormals u * 2^-24, which feed mma.sync.m16n8k16 directly as the A operand
//     (16 output channels x 16 k);
//   * the activations are the B operand (8 rows of x per MMA), staged once per CTA in
//     shared memory as binary16 hi + lo parts (x = hi + lo to ~2^-25 absolute) in the
//     k-order the nibble pairs come out in, so one 128-bit shared load feeds two MMAs;
//   * the "- 8" of the storage rule is folded into the accumulator's initial value
//     (-8 * sum of the group's x, computed once per CTA), and the group scale is
//     applied in f32 to each group's 32-term partial sum:
//        y = sum_groups s[n, g] * ( sum_{k in g} u[n,k] x[k]  -  8 sum_{k in g} x[k] ).
//     All products u*x are exact; accumulation is f32 in the tensor core and f32 FMA
//     across groups.  Dequantised weights are therefore never rounded at all in this
//     kernel; the bit-exact f32 expansion is a separate entry point sharing
//     kq::dequant_i4.
//   * K can be split across CTAs; partial sums go to the context workspace and the
//     last CTA to arrive for a row tile adds them in split order (deterministic).
//   * griddepcontrol lets the next launch start streaming its weights while this one
//     drains; nothing that depends on the previous kernel is touched before the wait.
//
// Activation domain: finite |x| <= 65504 (binary16 range).  Larger finite values raise
// the context's range flag, reported by the next kq_sync as KQ_ERR_RANGE.
#include <cmath>
#include <map>
#include <tuple>
#include <type_traits>

#include "kq_common.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kWarps = 8;               // row blocks (16 rows each) per CTA tile
constexpr int kTileRowsCta = kWarps * 16;
constexpr int kStages = 8;              // cp.async ring depth, chunks per warp
constexpr float kUnscale = 16777216.0f; // 2^24: undoes the subnormal encoding of the nibbles

struct GemvParams {
  const uint8_t* w[kMaxMulti];
  const float* bias[kMaxMulti];
  float* out[kMaxMulti];
  uint32_t n[kMaxMulti];
  uint32_t tile_begin[kMaxMulti + 1];
  uint32_t count;
  const void* x;
  uint32_t m, k;
  uint32_t chunks_per_split;
  uint32_t splits;
  uint32_t slab_chunks;  // chunks of x staged in shared memory at a time
  float* partial;        // [split][m][rows_total]
  uint32_t rows_total;
  unsigned int* counters;
  int* error_flag;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(__half lo, __half hi) {
  return static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
}

template <typename XT>
__device__ __forceinline__ void load_x8(const XT* p, float (&v)[8]) {
  if constexpr (std::is_same<XT, float>::value) {
    const float4 a = reinterpret_cast<const float4*>(p)[0];
    const float4 b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t parts[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same<XT, __half>::value) {
        v[2 * i] = __half2float(__ushort_as_half(static_cast<unsigned short>(parts[i] & 0xFFFFu)));
        v[2 * i + 1] = __half2float(__ushort_as_half(static_cast<unsigned short>(parts[i] >> 16)));
      } else {
        v[2 * i] = __uint_as_float(parts[i] << 16);
        v[2 * i + 1] = __uint_as_float(parts[i] & 0xFFFF0000u);
      }
    }
  }
}

// Stages groups [group0, group0 + groups) of x into shared memory.
//   xs_hi / xs_lo : [local group][kMT rows][32 halfs], the 8 values of each k-octet
//                   stored in the order 0,4,1,5,2,6,3,7
//   cpre          : [local group][kMT] f32 = -8 * 2^-24 * sum over the group of (hi + lo)
// Four consecutive threads share one (group, row): each converts one octet.
template <typename XT, int kMT, bool kHasLo>
__device__ __forceinline__ void stage_x(const XT* __restrict__ x, uint32_t m, uint32_t k,
                                        uint32_t group0, uint32_t groups, uint8_t* xs_hi,
                                        uint8_t* xs_lo, float* cpre, int* error_flag) {
  // rows that exist: one thread per (group, row, octet)
  const uint32_t items = groups * m * 4;
  const uint32_t items_padded = (items + 31u) & ~31u;  // whole warps run the shuffles below
  bool out_of_range = false;
  for (uint32_t item = threadIdx.x; item < items_padded; item += blockDim.x) {
    const bool valid = item < items;
    const uint32_t q = item & 3u;
    const uint32_t rest = item >> 2;
    const uint32_t row = rest % m;
    const uint32_t lg = rest / m;
    uint4 hi4 = make_uint4(0, 0, 0, 0), lo4 = make_uint4(0, 0, 0, 0);
    float sum = 0.0f;
    if (valid) {
      float v[8];
      load_x8<XT>(x + static_cast<size_t>(row) * k + (static_cast<size_t>(group0 + lg) << 5) + (q << 3), v);
      __half h[8], l[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float a = fabsf(v[e]);
        if (a > 65504.0f && a < __int_as_float(0x7f800000)) out_of_range = true;
        h[e] = __float2half_rn(v[e]);
        const float hf = __half2float(h[e]);
        if constexpr (kHasLo) {
          l[e] = __float2half_rn(v[e] - hf);
          sum += hf + __half2float(l[e]);
        } else {
          sum += hf;
        }
      }
      hi4 = make_uint4(pack_half2(h[0], h[4]), pack_half2(h[1], h[5]), pack_half2(h[2], h[6]),
                       pack_half2(h[3], h[7]));
      if constexpr (kHasLo)
        lo4 = make_uint4(pack_half2(l[0], l[4]), pack_half2(l[1], l[5]), pack_half2(l[2], l[6]),
                         pack_half2(l[3], l[7]));
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (valid) {
      const uint32_t off = lg * (kMT * 64) + row * 64 + q * 16;
      *reinterpret_cast<uint4*>(xs_hi + off) = hi4;
      if constexpr (kHasLo) *reinterpret_cast<uint4*>(xs_lo + off) = lo4;
      if (q == 0) cpre[lg * kMT + row] = sum * (-8.0f / kUnscale);
    }
  }
  // rows of the MMA tile beyond m: zeros (their output columns are never stored)
  const uint32_t pad_rows = kMT - m;
  for (uint32_t item = threadIdx.x; item < groups * pad_rows * 4; item += blockDim.x) {
    const uint32_t q = item & 3u;
    const uint32_t rest = item >> 2;
    const uint32_t row = m + rest % pad_rows;
    const uint32_t lg = rest / pad_rows;
    const uint32_t off = lg * (kMT * 64) + row * 64 + q * 16;
    *reinterpret_cast<uint4*>(xs_hi + off) = make_uint4(0, 0, 0, 0);
    if constexpr (kHasLo) *reinterpret_cast<uint4*>(xs_lo + off) = make_uint4(0, 0, 0, 0);
    if (q == 0) cpre[lg * kMT + row] = 0.0f;
  }
  if (out_of_range) *reinterpret_cast<volatile int*>(error_flag) = 1;  // sticky, host-mapped word
}

template <typename XT, bool kScaleF16, int kMT>
__global__ void __launch_bounds__(kWarps * 32)
qgemv_i4_kernel(const GemvParams p) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;  // chunk bytes
  constexpr int kTiles = kMT / 8;

  extern __shared__ __align__(16) uint8_t smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;

  pdl_launch_dependents();

  // which weight of the launch this CTA's row tile belongs to
  uint32_t wi = 0;
#pragma unroll
  for (int i = 1; i < kMaxMulti; ++i)
    if (i < static_cast<int>(p.count) && blockIdx.x >= p.tile_begin[i]) wi = i;
  const uint8_t* w_base = p.w[0];
  const float* bias = p.bias[0];
  float* out = p.out[0];
  uint32_t n = p.n[0], tile0 = p.tile_begin[0];
#pragma unroll
  for (int i = 1; i < kMaxMulti; ++i)
    if (wi == static_cast<uint32_t>(i)) {
      w_base = p.w[i]; bias = p.bias[i]; out = p.out[i]; n = p.n[i]; tile0 = p.tile_begin[i];
    }
  const uint32_t tile = blockIdx.x - tile0;
  const uint32_t row_block = tile * kWarps + warp;
  const bool active = row_block * 16u < n;

  const uint32_t chunks_per_row = p.k / kChunkK;
  const uint32_t split = blockIdx.y;
  const uint32_t cbeg = split * p.chunks_per_split;
  const uint32_t cend = min(cbeg + p.chunks_per_split, chunks_per_row);
  const uint32_t nch = cend - cbeg;

  uint8_t* ring = smem + warp * (kStages * kCB);
  const uint32_t slab_groups = 2 * p.slab_chunks;
  uint8_t* xs_hi = smem + kWarps * kStages * kCB;
  uint8_t* xs_lo = xs_hi + (kHasLo ? slab_groups * kMT * 64 : 0);
  float* cpre = reinterpret_cast<float*>(xs_lo + slab_groups * kMT * 64);

  const uint8_t* stream = w_base + (static_cast<size_t>(row_block) * chunks_per_row + cbeg) * kCB;

  auto issue = [&](uint32_t c) {
    const uint8_t* src = stream + static_cast<size_t>(c) * kCB;
    uint8_t* dst = ring + (c % kStages) * kCB;
    cp_async16(dst + lane * 16, src + lane * 16);
    if (lane < 2 * kScaleBytes) cp_async16(dst + kChunkWeightBytes + lane * 16, src + kChunkWeightBytes + lane * 16);
  };

  // Weights do not depend on the previous kernel: start streaming before the wait.
#pragma unroll
  for (int s = 0; s < kStages; ++s) {
    if (active && static_cast<uint32_t>(s) < nch) issue(s);
    cp_async_commit();
  }

  pdl_wait_prior_grid();

  float acc[kTiles][4];
#pragma unroll
  for (int i = 0; i < kTiles; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  const XT* x = static_cast<const XT*>(p.x);
  constexpr uint32_t kMask = 0x000F000Fu;

  uint32_t in_slab = 0;
  for (uint32_t c = 0; c < nch; ++c, ++in_slab) {
    if (in_slab == p.slab_chunks) in_slab = 0;
    if (in_slab == 0) {
      if (c != 0) __syncthreads();  // everyone is done reading the previous slab
      const uint32_t chunks_here = min(p.slab_chunks, nch - c);
      stage_x<XT, kMT, kHasLo>(x, p.m, p.k, 2 * (cbeg + c), 2 * chunks_here, xs_hi, xs_lo, cpre,
                               p.error_flag);
      __syncthreads();
    }
    cp_async_wait<kStages - 1>();
    __syncwarp();
    if (active) {
      const uint8_t* slot = ring + (c % kStages) * kCB;
      const uint4 wq = *reinterpret_cast<const uint4*>(slot + lane * 16);
      float sc[4];  // {row g, grp 0}, {row g+8, grp 0}, {row g, grp 1}, {row g+8, grp 1}
      if constexpr (kScaleF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>(slot + kChunkWeightBytes + g * 8);
        sc[0] = __half2float(__ushort_as_half(static_cast<unsigned short>(raw.x & 0xFFFFu)));
        sc[1] = __half2float(__ushort_as_half(static_cast<unsigned short>(raw.x >> 16)));
        sc[2] = __half2float(__ushort_as_half(static_cast<unsigned short>(raw.y & 0xFFFFu)));
        sc[3] = __half2float(__ushort_as_half(static_cast<unsigned short>(raw.y >> 16)));
      } else {
        const float4 raw = *reinterpret_cast<const float4*>(slot + kChunkWeightBytes + g * 16);
        sc[0] = raw.x; sc[1] = raw.y; sc[2] = raw.z; sc[3] = raw.w;
      }
      __syncwarp();  // the slot is free once every lane has read it
      if (c + kStages < nch) issue(c + kStages);
      cp_async_commit();

#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const uint32_t wa = jj ? wq.z : wq.x;  // row g
        const uint32_t wb = jj ? wq.w : wq.y;  // row g + 8
        // nibble pairs (e, e+4) of the lane's k-octet, as binary16 subnormals u * 2^-24
        const uint32_t a0[4] = {wa & kMask, wb & kMask, (wa >> 4) & kMask, (wb >> 4) & kMask};
        const uint32_t a1[4] = {(wa >> 8) & kMask, (wb >> 8) & kMask, (wa >> 12) & kMask, (wb >> 12) & kMask};
        const uint32_t lg = 2 * in_slab + jj;
#pragma unroll
        for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
          const uint32_t off = lg * (kMT * 64) + tile_m * 512 + lane * 16;
          const uint4 bh = *reinterpret_cast<const uint4*>(xs_hi + off);
          const float2 c0 = *reinterpret_cast<const float2*>(cpre + lg * kMT + tile_m * 8 + 2 * t);
          float cf[4] = {c0.x, c0.y, c0.x, c0.y};
          mma_f16(cf, a0, bh.x, bh.y);
          mma_f16(cf, a1, bh.z, bh.w);
          if constexpr (kHasLo) {
            const uint4 bl = *reinterpret_cast<const uint4*>(xs_lo + off);
            mma_f16(cf, a0, bl.x, bl.y);
            mma_f16(cf, a1, bl.z, bl.w);
          }
          acc[tile_m][0] = fmaf(sc[2 * jj], cf[0], acc[tile_m][0]);
          acc[tile_m][1] = fmaf(sc[2 * jj], cf[1], acc[tile_m][1]);
          acc[tile_m][2] = fmaf(sc[2 * jj + 1], cf[2], acc[tile_m][2]);
          acc[tile_m][3] = fmaf(sc[2 * jj + 1], cf[3], acc[tile_m][3]);
        }
      }
    } else {
      cp_async_commit();
    }
  }
  cp_async_wait<0>();

  // ---- epilogue -----------------------------------------------------------------
  const uint32_t row_a = row_block * 16u + g;
  if (p.splits == 1) {
    if (active) {
      const float bias_a = bias[row_a], bias_b = bias[row_a + 8];
#pragma unroll
      for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t mm = tile_m * 8 + 2 * t + j;
          if (mm < p.m) {
            out[static_cast<size_t>(mm) * n + row_a] = fmaf(acc[tile_m][j], kUnscale, bias_a);
            out[static_cast<size_t>(mm) * n + row_a + 8] = fmaf(acc[tile_m][2 + j], kUnscale, bias_b);
          }
        }
      }
    }
    return;
  }

  const uint32_t ws_row0 = blockIdx.x * kTileRowsCta;  // this tile's first row in the workspace
  if (active) {
    float* part = p.partial + static_cast<size_t>(split) * p.m * p.rows_total;
    const uint32_t r = ws_row0 + warp * 16u + g;
#pragma unroll
    for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t mm = tile_m * 8 + 2 * t + j;
        if (mm < p.m) {
          __stcg(part + static_cast<size_t>(mm) * p.rows_total + r, acc[tile_m][j]);
          __stcg(part + static_cast<size_t>(mm) * p.rows_total + r + 8, acc[tile_m][2 + j]);
        }
      }
    }
  }
  __shared__ unsigned int arrival;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) arrival = atomicAdd(p.counters + blockIdx.x, 1u);
  __syncthreads();
  if (arrival != p.splits - 1) return;
  __threadfence();
  // Last CTA of this row tile: add the partial sums in split order.
  const uint32_t rows_here = min(static_cast<uint32_t>(kTileRowsCta), n - tile * kTileRowsCta);
  for (uint32_t idx = threadIdx.x; idx < rows_here * p.m; idx += blockDim.x) {
    const uint32_t mm = idx / rows_here, r = idx % rows_here;
    float total = 0.0f;
    for (uint32_t s = 0; s < p.splits; ++s)
      total += __ldcg(p.partial + (static_cast<size_t>(s) * p.m + mm) * p.rows_total + ws_row0 + r);
    const uint32_t row = tile * kTileRowsCta + r;
    out[static_cast<size_t>(mm) * n + row] = fmaf(total, kUnscale, bias[row]);
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;  // ready for the next launch
}

template <typename XT, bool kScaleF16, int kMT>
size_t smem_bytes(uint32_t slab_chunks) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  const size_t cb = kChunkWeightBytes + 32u * (kScaleF16 ? 2u : 4u);
  const size_t groups = 2 * slab_chunks;
  return kWarps * kStages * cb + groups * kMT * 64 * (kHasLo ? 2 : 1) + groups * kMT * 4;
}

struct Plan {
  uint32_t splits, chunks_per_split, slab_chunks;
};

template <typename XT, bool kScaleF16, int kMT>
cudaError_t launch_typed(const LaunchEnv& env, GemvParams& p, uint32_t tiles) {
  auto kernel = qgemv_i4_kernel<XT, kScaleF16, kMT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const uint32_t chunks_per_row = p.k / kChunkK;
  const uint32_t slab_cap = kMT == 8 ? 32u : 16u;

  // Split K until the grid fills the machine; a pure function of the shape (never
  // autotuned), memoised because the occupancy queries are host-side work.
  static std::map<std::tuple<uint32_t, uint32_t, uint32_t, uint64_t>, Plan> cache;
  const auto key = std::make_tuple(tiles, chunks_per_row, p.m, env.workspace_bytes);
  auto hit = cache.find(key);
  Plan best{1, chunks_per_row, std::min(chunks_per_row, slab_cap)};
  if (hit != cache.end()) {
    best = hit->second;
  } else {
    double best_cost = 1e30;
    const uint32_t max_splits = std::min<uint32_t>(32u, chunks_per_row);
    for (uint32_t s = 1; s <= max_splits; ++s) {
      const uint32_t cps = (chunks_per_row + s - 1) / s;
      const uint32_t real = (chunks_per_row + cps - 1) / cps;
      if (real != s) continue;
      const uint32_t slab = std::min(cps, slab_cap);
      if (s > 1) {
        const uint64_t need = static_cast<uint64_t>(s) * p.m * p.rows_total * sizeof(float);
        if (need > env.workspace_bytes || tiles > env.counter_count) continue;
      }
      int per_sm = 0;
      cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
          &per_sm, kernel, kWarps * 32, smem_bytes<XT, kScaleF16, kMT>(slab));
      if (e != cudaSuccess) return e;
      if (per_sm < 1) continue;
      const double slots = static_cast<double>(env.sm_count) * per_sm;
      const double waves = std::ceil(static_cast<double>(tiles) * s / slots);
      const double cost = waves * (cps + 6.0) + (s > 1 ? 1.0 : 0.0);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best = Plan{s, cps, slab};
      }
    }
    if (best_cost > 1e29) return cudaErrorInvalidConfiguration;
    cache.emplace(key, best);
  }
  p.splits = best.splits;
  p.chunks_per_split = best.chunks_per_split;
  p.slab_chunks = best.slab_chunks;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, best.splits, 1);
  cfg.blockDim = dim3(kWarps * 32, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes<XT, kScaleF16, kMT>(best.slab_chunks);
  cfg.stream = env.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = env.overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

template <typename XT>
cudaError_t launch_x(const LaunchEnv& env, GemvParams& p, uint32_t tiles, bool scale_f16) {
  if (p.m <= 8) {
    return scale_f16 ? launch_typed<XT, true, 8>(env, p, tiles) : launch_typed<XT, false, 8>(env, p, tiles);
  }
  return scale_f16 ? launch_typed<XT, true, 16>(env, p, tiles) : launch_typed<XT, false, 16>(env, p, tiles);
}

}  // namespace

bool qgemv_i4_supports(const Weight& w, uint32_t m) {
  return w.layout == kLayoutTiledI4 && m >= 1 && m <= 16;
}

cudaError_t launch_qgemv_i4(const LaunchEnv& env, int count, const LinearTarget* targets,
                            const void* x, int x_dtype, uint32_t m, int* launches) {
  if (count < 1 || count > kMaxMulti) return cudaErrorInvalidValue;
  GemvParams p = {};
  p.count = static_cast<uint32_t>(count);
  uint32_t tiles = 0;
  const uint32_t k = targets[0].w->k;
  const int scale_dtype = targets[0].w->scale_dtype;
  for (int i = 0; i < count; ++i) {
    const Weight& w = *targets[i].w;
    if (w.layout != kLayoutTiledI4 || w.k != k || w.scale_dtype != scale_dtype) return cudaErrorInvalidValue;
    p.w[i] = static_cast<const uint8_t*>(w.data);
    p.bias[i] = targets[i].bias;
    p.out[i] = targets[i].out;
    p.n[i] = w.n;
    p.tile_begin[i] = tiles;
    tiles += (w.n + kTileRowsCta - 1) / kTileRowsCta;
  }
  for (int i = count; i <= kMaxMulti; ++i) p.tile_begin[i] = tiles;
  p.x = x;
  p.m = m;
  p.k = k;
  p.partial = static_cast<float*>(env.workspace);
  p.rows_total = tiles * kTileRowsCta;
  p.counters = env.counters;
  p.error_flag = env.error_flag;
  const bool f16s = scale_dtype == KQ_F16;
  cudaError_t e;
  switch (x_dtype) {
    case KQ_F32: e = launch_x<float>(env, p, tiles, f16s); break;
    case KQ_F16: e = launch_x<__half>(env, p, tiles, f16s); break;
    case KQ_BF16: e = launch_x<__nv_bfloat16>(env, p, tiles, f16s); break;
    default: return cudaErrorInvalidValue;
  }
  if (e == cudaSuccess && launches) *launches += 1;
  return e;
}

}  // namespace kq
