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
//   * each lane streams its weights with 128-bit read-only loads straight into a
//     register ring (kDepth chunks ahead per row block); weights never touch shared
//     memory, whose bandwidth the activations need;
//   * a nibble is never converted: `word & 0x000F000F` IS a pair of binary16
//     subnormals u * 2^-24 and `word & 0x00F000F0` a pair u * 2^-20; both feed
//     mma.sync.m16n8k16 directly as the A operand (16 output channels x 16 k), the
//     factor 16 being taken out of the matching activations when they are staged.
//     Integer/logic instructions issue at half rate, so the unpack (5 per 8 weights)
//     is the scarce resource of the whole kernel;
//   * the activations are the B operand.  They are staged once per CTA in shared
//     memory as binary16 in the k-order the nibble pairs come out in, so one 128-bit
//     shared load feeds two MMAs and is reused by both row blocks of the warp.  f32 and
//     bf16 activations are split as x = hi + lo (binary16 each, after the power-of-two
//     pre-scale of their group: ~2^-22 of the value) and
//     the two parts sit in ADJACENT columns of the same MMA tile, so the extra
//     precision costs no extra MMA: the lane that owns column pair (2t, 2t+1) adds the
//     two partial sums;
//   * the "- 8" of the storage rule is folded into the accumulator's initial value
//     (-8 * sum of the group's x, computed once per CTA), and the group scale is
//     applied in f32 to each group's 32-term partial sum:
//        y = sum_groups s[n, g] * ( sum_{k in g} u[n,k] x[k]  -  8 sum_{k in g} x[k] ).
//     All products u*x are exact; accumulation is f32 in the tensor core and f32 FMA
//     across groups.  Dequantised weights are therefore never rounded at all in this
//     kernel; the bit-exact f32 expansion is a separate entry point sharing
//     kq::dequant_i4.
//   * K can be split across the CTAs of a thread-block cluster (up to 8); each CTA
//     leaves its partial sums in its own shared memory and, after one cluster barrier,
//     every CTA adds a slice of the rows over distributed shared memory in rank order
//     (deterministic, no global scratch, no atomics).
//   * griddepcontrol lets the next launch start streaming its weights while this one
//     drains; nothing that depends on the previous kernel is touched before the wait.
//
// Activation domain: any f32 / binary16 / bfloat16 value.  Every 32-k group of an activation
// row (every whole row in the wide kernel) is pre-scaled by an exact power of two before it is
// split into binary16 parts, and the inverse is applied to the group's partial sum in f32
// (kq_gemv_core.cuh: pow2_prescale), so the result does not depend on the magnitude of x.
#include <algorithm>
#include <type_traits>

#include "kq_gemv_core.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kWarps = 4;                // warps per CTA
constexpr int kDepth = 4;                // chunks in flight per row block, in registers
constexpr uint32_t kWantCtasPerSm = 4;   // K is split over a cluster until the grid offers this many CTAs per SM
constexpr uint32_t kWideSlabBytes = 16384;  // staged activations per column tile the wide kernel holds at a time
constexpr int kMaxCluster = 8;           // portable cluster size: K splits per row tile

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
  // Activations already converted to the staged layout by stage_x_global_kernel (wide kernel
  // only; null: every CTA converts its own slab).
  const uint8_t* staged_xs;
  const float* staged_corr;
  const float* staged_inv;  // [m]: 2^-e of every activation row (wide kernel)
  const float* residual;    // null, or [m, n] added to the single output (wide kernel; may alias the output)
  // Non-null: a row-parallel shard; the outputs are added across ranks in the epilogue.
  const FusedCommDev* fcomm;
};

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// K was split over the CTAs of a cluster: every CTA holds its partial sums in `red`
// ([m][tile_rows] f32 in its own shared memory); after one cluster barrier each CTA adds a
// slice of the tile's outputs over distributed shared memory, ranks in ascending order.
__device__ __forceinline__ void cluster_reduce_store(const GemvParams& p, float* red, uint32_t tile_rows,
                                                     uint32_t tile, uint32_t split, uint32_t n, float* out,
                                                     const float* bias) {
  cluster_sync_all();
  const uint32_t rows_here = min(tile_rows, n - tile * tile_rows);
  const uint32_t total = rows_here * p.m;
  const uint32_t per_rank = (total + p.splits - 1) / p.splits;
  const uint32_t lo = min(split * per_rank, total), hi = min(lo + per_rank, total);
  const uint32_t red_base = static_cast<uint32_t>(__cvta_generic_to_shared(red));
  for (uint32_t idx = lo + threadIdx.x; idx < hi; idx += blockDim.x) {
    const uint32_t mm = idx / rows_here, r = idx - mm * rows_here;
    const uint32_t local = red_base + (mm * tile_rows + r) * 4u;
    float sum = 0.0f;
    for (uint32_t s = 0; s < p.splits; ++s) sum += ld_cluster_f32(cluster_map_shared(local, s));
    const uint32_t row = tile * tile_rows + r;
    float v = fmaf(sum, kUnscale, bias[row]);
    if (p.residual != nullptr) v = __fadd_rn(v, p.residual[static_cast<size_t>(mm) * n + row]);
    out[static_cast<size_t>(mm) * n + row] = v;
  }
  cluster_sync_all();  // nobody's shared memory may go away while a peer still reads it
}

constexpr uint32_t kFusedSpinLimit = 1u << 22;

// One exchange entry = {value, epoch} in ONE aligned 64-bit word, written and polled with
// scalar 64-bit accesses: those are single-copy atomic, so a reader that sees the new epoch
// also sees the value that was stored with it (a two-word vector access gives no such
// guarantee).  Relaxed, system scope: the entry carries its own flag, nothing else is ordered.
__device__ __forceinline__ void st_entry(uint2* p, float value, unsigned int epoch) {
  const unsigned long long word = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(value);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(word) : "memory");
}
__device__ __forceinline__ uint2 ld_entry(const uint2* p) {
  unsigned long long word;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(p) : "memory");
  return make_uint2(static_cast<uint32_t>(word), static_cast<uint32_t>(word >> 32));
}

// Row-parallel shard: the tile's outputs (partial sums over this rank's k range, in `red`,
// possibly spread over the CTAs of a cluster) are added across ranks here, CTA by CTA:
//   1. every thread finishes its few outputs and PUSHES each into every peer's exchange area
//      (slot = epoch parity, source = this rank) as one 8-byte store {value, epoch};
//   2. it then polls (bounded) its own area until the peers' entries carry this epoch;
//   3. and adds the ranks' values in rank order (all ranks get the same bits) plus the bias.
// A CTA depends only on its twins on the other GPUs, which run the same grid, so nothing
// waits on a CTA that is not resident as long as the grid fits the GPU in one wave (the host
// checks).  The last CTA to finish advances the epoch for the next launch.
__device__ __forceinline__ void reduce_exchange_store(const GemvParams& p, float* red, uint32_t tile_rows,
                                                      uint32_t tile, uint32_t split, uint32_t n, float* out,
                                                      const float* bias, unsigned int epoch) {
  const FusedCommDev& fc = *p.fcomm;
  const uint32_t me = fc.rank, world = fc.world;
  if (p.splits > 1) cluster_sync_all();
  else __syncthreads();
  const uint32_t rows_here = min(tile_rows, n - tile * tile_rows);
  const uint32_t total = rows_here * p.m;
  const uint32_t per_rank = (total + p.splits - 1) / p.splits;
  const uint32_t lo = min(split * per_rank, total), hi = min(lo + per_rank, total);
  const uint32_t red_base = static_cast<uint32_t>(__cvta_generic_to_shared(red));
  constexpr int kMaxPer = 4;  // tile_rows * m / threads <= 64 * 4 / 128, with room to spare
  float v[kMaxPer];
  uint32_t off[kMaxPer], rowi[kMaxPer];
  int cnt = 0;
  for (uint32_t idx = lo + threadIdx.x; idx < hi && cnt < kMaxPer; idx += blockDim.x) {
    const uint32_t mm = idx / rows_here, r = idx - mm * rows_here;
    float sum = 0.0f;
    if (p.splits > 1) {
      const uint32_t local = red_base + (mm * tile_rows + r) * 4u;
      for (uint32_t s = 0; s < p.splits; ++s) sum += ld_cluster_f32(cluster_map_shared(local, s));
    } else {
      sum = red[mm * tile_rows + r];
    }
    const uint32_t row = tile * tile_rows + r;
    v[cnt] = sum * kUnscale;
    off[cnt] = mm * n + row;
    rowi[cnt] = row;
    ++cnt;
  }
  // Low-latency exchange: every output travels as one aligned 8-byte store {value, epoch}, so
  // data and flag arrive together and no fence or separate flag is needed; the receiver polls
  // the entry itself.  Entries of consecutive epochs alternate between two slots, so a peer
  // that is one exchange ahead never overwrites an entry that has not been read.
  const uint32_t parity = epoch & 1u;
  const uint64_t slot_entries = kFusedSlotBytes / 8;
  for (uint32_t r = 0; r < world; ++r) {
    if (r == me) continue;
    uint2* dst = reinterpret_cast<uint2*>(fc.base[r] + fc.data_off) + (static_cast<uint64_t>(parity) * kFusedMaxWorld + me) * slot_entries;
    for (int i = 0; i < cnt; ++i)
      st_entry(dst + off[i], v[i], epoch);
  }
  for (int i = 0; i < cnt; ++i) {
    float sum = 0.0f;
    for (uint32_t r = 0; r < world; ++r) {
      if (r == me) {
        sum += v[i];
        continue;
      }
      const uint2* src = reinterpret_cast<const uint2*>(fc.base[me] + fc.data_off) +
                         (static_cast<uint64_t>(parity) * kFusedMaxWorld + r) * slot_entries + off[i];
      uint2 e;
      uint32_t spins = 0;
      while (true) {
        e = ld_entry(src);
        if (e.y == epoch) break;
        if (++spins > kFusedSpinLimit) {
          *reinterpret_cast<volatile int*>(fc.status) = 1;
          break;
        }
      }
      sum += __uint_as_float(e.x);
    }
    out[off[i]] = sum + bias[rowi[i]];
  }
  if (p.splits > 1) cluster_sync_all();  // nobody's shared memory may go away while a peer still reads it
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int finished = atomicAdd(fc.done, 1u) + 1u;
    if (finished == gridDim.x * gridDim.y) {
      *reinterpret_cast<volatile unsigned int*>(fc.done) = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(fc.epoch) = epoch;
    }
  }
}

template <bool kScaleF16>
struct ChunkRegs {
  uint4 w;  // row g grp 0 | row g+8 grp 0 | row g grp 1 | row g+8 grp 1
  typename std::conditional<kScaleF16, uint2, uint4>::type s;
};
template <typename XT, bool kScaleF16, int kCols, int kRB>
__global__ void __launch_bounds__(kWarps * 32)
qgemv_i4_kernel(const GemvParams p) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;  // chunk bytes
  constexpr int kTiles = kCols / 8;
  constexpr int kAccPerTile = kHasLo ? 2 : 4;
  constexpr int kCorrPerTile = kHasLo ? 1 : 2;
  constexpr int kCorrStride = kHasLo ? kCols / 2 : kCols;
  constexpr uint32_t kTileRowsCta = kWarps * kRB * 16;

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
  const uint32_t row_block0 = (tile * kWarps + warp) * kRB;

  const uint32_t chunks_per_row = p.k / kChunkK;
  const uint32_t split = blockIdx.y;  // == rank in the cluster when splits > 1
  const uint32_t cbeg = min(split * p.chunks_per_split, chunks_per_row);
  const uint32_t cend = min(cbeg + p.chunks_per_split, chunks_per_row);
  const uint32_t nch = cend - cbeg;

  const uint32_t active_cols = kHasLo ? 2 * p.m : p.m;
  const uint32_t xs_stride = active_cols * 64;  // bytes of staged activations per group
  uint8_t* xs = smem;
  float* corr = reinterpret_cast<float*>(smem + 2 * p.slab_chunks * xs_stride);

  bool active[kRB];
  const uint8_t* next[kRB];  // address this lane loads for the chunk kDepth ahead of the current block
#pragma unroll
  for (int r = 0; r < kRB; ++r) {
    active[r] = (row_block0 + r) * 16u < n;
    next[r] = w_base + (static_cast<size_t>(row_block0 + r) * chunks_per_row + cbeg) * kCB + lane * 16;
  }
  const uint32_t scale_off = kChunkWeightBytes - lane * 16 + g * (4 * kScaleBytes);

  ChunkRegs<kScaleF16> ring[kDepth][kRB];
  auto fetch = [&](ChunkRegs<kScaleF16>& dst, const uint8_t* src) {
    dst.w = ldg_stream_v4(src);
    if constexpr (kScaleF16) dst.s = ldg_stream_v2(src + scale_off);
    else dst.s = ldg_stream_v4(src + scale_off);
  };

  // Weights do not depend on the previous kernel: start streaming before the wait.
#pragma unroll
  for (int d = 0; d < kDepth; ++d)
#pragma unroll
    for (int r = 0; r < kRB; ++r) {
      ring[d][r].w = make_uint4(0, 0, 0, 0);
      if constexpr (kScaleF16) ring[d][r].s = make_uint2(0, 0);
      else ring[d][r].s = make_uint4(0, 0, 0, 0);
      if (active[r] && static_cast<uint32_t>(d) < nch) fetch(ring[d][r], next[r] + d * kCB);
    }
#pragma unroll
  for (int r = 0; r < kRB; ++r) next[r] += kDepth * kCB;

  pdl_wait_prior_grid();

  float acc[kRB][kTiles][kAccPerTile];
#pragma unroll
  for (int r = 0; r < kRB; ++r)
#pragma unroll
    for (int i = 0; i < kTiles; ++i)
#pragma unroll
      for (int j = 0; j < kAccPerTile; ++j) acc[r][i][j] = 0.0f;

  const XT* x = static_cast<const XT*>(p.x);
  constexpr uint32_t kMask0 = 0x000F000Fu;  // nibbles 0 and 4 of a word: u * 2^-24 as binary16
  constexpr uint32_t kMask1 = 0x00F000F0u;  // nibbles 1 and 5 of a word: u * 2^-20 as binary16

  // B fragments and "-8 sum x" terms live in registers that only lanes with a real
  // column / activation row ever load into; everybody else keeps the initial zeros.
  uint4 bfrag[kTiles];
  float cterm[kTiles][kCorrPerTile], cinv[kTiles][kCorrPerTile];  // {-8 sum x, 2^-e} of the lane's activation rows
  bool load_b[kTiles], load_c[kTiles][kCorrPerTile];
#pragma unroll
  for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
    bfrag[tile_m] = make_uint4(0, 0, 0, 0);
    load_b[tile_m] = tile_m * 8 + g < active_cols;
#pragma unroll
    for (int j = 0; j < kCorrPerTile; ++j) {
      cterm[tile_m][j] = 0.0f;
      cinv[tile_m][j] = 0.0f;
      const uint32_t mm = kHasLo ? tile_m * 4 + t : tile_m * 8 + 2 * t + j;
      load_c[tile_m][j] = mm < p.m;
    }
  }
  const uint32_t xs_lane = static_cast<uint32_t>(__cvta_generic_to_shared(xs)) + lane * 16;
  const uint32_t corr_lane = static_cast<uint32_t>(__cvta_generic_to_shared(corr)) + (kHasLo ? t : 2 * t) * 8;

  // One chunk (64 k = two scale groups) of every row block of the warp, out of ring
  // slot d; then the slot is refilled with the chunk kDepth further on.
  auto process = [&](const int d, uint32_t xs_addr, uint32_t corr_addr, bool refill) {
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
#pragma unroll
      for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
        lds_v4_if(bfrag[tile_m], xs_addr + jj * xs_stride + tile_m * 512, load_b[tile_m]);
#pragma unroll
        for (int j = 0; j < kCorrPerTile; ++j)
          lds_v2f_if(cterm[tile_m][j], cinv[tile_m][j], corr_addr + (jj * kCorrStride + tile_m * (kHasLo ? 4 : 8) + j) * 8,
                     load_c[tile_m][j]);
      }
#pragma unroll
      for (int r = 0; r < kRB; ++r) {
        const uint32_t wa = jj ? ring[d][r].w.z : ring[d][r].w.x;  // row g
        const uint32_t wb = jj ? ring[d][r].w.w : ring[d][r].w.y;  // row g + 8
        const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
        const uint32_t a0[4] = {wa & kMask0, wb & kMask0, wa & kMask1, wb & kMask1};
        const uint32_t a1[4] = {wa8 & kMask0, wb8 & kMask0, wa8 & kMask1, wb8 & kMask1};
        float2 s;  // .x = row g, .y = row g + 8
        if constexpr (kScaleF16) {
          s = __half22float2(*reinterpret_cast<const __half2*>(jj ? &ring[d][r].s.y : &ring[d][r].s.x));
        } else {
          s = jj ? make_float2(__uint_as_float(ring[d][r].s.z), __uint_as_float(ring[d][r].s.w))
                 : make_float2(__uint_as_float(ring[d][r].s.x), __uint_as_float(ring[d][r].s.y));
        }
#pragma unroll
        for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
          float cf[4];
          mma_f16_zero(cf, a0, bfrag[tile_m].x, bfrag[tile_m].y);
          mma_f16(cf, a1, bfrag[tile_m].z, bfrag[tile_m].w);
          if constexpr (kHasLo) {
            acc[r][tile_m][0] = fmaf(s.x, fmaf(cf[0] + cf[1], cinv[tile_m][0], cterm[tile_m][0]), acc[r][tile_m][0]);
            acc[r][tile_m][1] = fmaf(s.y, fmaf(cf[2] + cf[3], cinv[tile_m][0], cterm[tile_m][0]), acc[r][tile_m][1]);
          } else {
            acc[r][tile_m][0] = fmaf(s.x, fmaf(cf[0], cinv[tile_m][0], cterm[tile_m][0]), acc[r][tile_m][0]);
            acc[r][tile_m][1] = fmaf(s.x, fmaf(cf[1], cinv[tile_m][1], cterm[tile_m][1]), acc[r][tile_m][1]);
            acc[r][tile_m][2] = fmaf(s.y, fmaf(cf[2], cinv[tile_m][0], cterm[tile_m][0]), acc[r][tile_m][2]);
            acc[r][tile_m][3] = fmaf(s.y, fmaf(cf[3], cinv[tile_m][1], cterm[tile_m][1]), acc[r][tile_m][3]);
          }
        }
      }
    }
    if (refill) {
#pragma unroll
      for (int r = 0; r < kRB; ++r)
        if (active[r]) fetch(ring[d][r], next[r] + d * kCB);
    }
  };

  for (uint32_t done = 0; done < nch;) {
    const uint32_t slab_n = min(p.slab_chunks, nch - done);
    if (done != 0) __syncthreads();  // everyone is done reading the previous slab
    stage_x<XT, kHasLo, kCorrStride>(x, p.m, p.k, 2 * (cbeg + done), 2 * slab_n, xs, xs_stride, corr);
    __syncthreads();
    uint32_t xs_addr = xs_lane, corr_addr = corr_lane;
    uint32_t i = 0;
    for (; i + kDepth <= slab_n; i += kDepth) {
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        process(d, xs_addr, corr_addr, done + i + d + kDepth < nch);
        xs_addr += 2 * xs_stride;
        corr_addr += 2 * kCorrStride * 8;
      }
#pragma unroll
      for (int r = 0; r < kRB; ++r) next[r] += kDepth * kCB;
    }
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d) {  // the last, short block of the split
      if (i + d < slab_n) {
        process(d, xs_addr, corr_addr, false);
        xs_addr += 2 * xs_stride;
        corr_addr += 2 * kCorrStride * 8;
      }
    }
    done += slab_n;
  }

  // ---- epilogue -----------------------------------------------------------------
  // lane owns, per row block and tile: rows g and g+8 of the block and activation rows
  //   with hi/lo columns : mm = 4*tile + t             (acc[..][0] row g, [1] row g+8)
  //   binary16 input     : mm = 8*tile + 2t, 2t+1      (acc[..][0,1] row g, [2,3] row g+8)
  float* red = reinterpret_cast<float*>(smem);  // [m][kTileRowsCta], aliases the x slab
  if (p.splits > 1) __syncthreads();            // the slab is dead from here on
#pragma unroll
  for (int r = 0; r < kRB; ++r) {
    if (!active[r]) continue;
    const uint32_t row_a = (row_block0 + r) * 16u + g;
    const uint32_t tr_a = (warp * kRB + r) * 16u + g;  // row inside the CTA tile
    float bias_a = 0.0f, bias_b = 0.0f;
    if (p.splits == 1) {
      bias_a = bias[row_a];
      bias_b = bias[row_a + 8];
    }
#pragma unroll
    for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
#pragma unroll
      for (int j = 0; j < (kHasLo ? 1 : 2); ++j) {
        const uint32_t mm = kHasLo ? tile_m * 4 + t : tile_m * 8 + 2 * t + j;
        if (mm >= p.m) continue;
        const float va = acc[r][tile_m][kHasLo ? 0 : j];
        const float vb = acc[r][tile_m][kHasLo ? 1 : 2 + j];
        if (p.splits == 1) {
          out[static_cast<size_t>(mm) * n + row_a] = fmaf(va, kUnscale, bias_a);
          out[static_cast<size_t>(mm) * n + row_a + 8] = fmaf(vb, kUnscale, bias_b);
        } else {
          red[mm * kTileRowsCta + tr_a] = va;
          red[mm * kTileRowsCta + tr_a + 8] = vb;
        }
      }
    }
  }
  if (p.splits == 1) return;

  cluster_reduce_store(p, red, kTileRowsCta, tile, split, n, out, bias);
}

// ---- group-packed variant: at most 4 of the 8 MMA columns are needed -----------------
// With one or two activation rows the block above would leave most of each MMA tile empty
// and, worse, make every lane apply every group's scale.  Here the spare columns carry
// OTHER scale groups: a unit is kG consecutive groups, group j of the unit owns columns
// [j * kCpg, (j + 1) * kCpg) of the tile (its activations are zero in every other column),
// and the 2 * kG MMAs of the unit accumulate into ONE C tile.  Column block j of C then
// holds group j's partial sums only, so a lane scales just the group its two C columns
// belong to: one scale pair, one "-8 sum x" term and three FP instructions per row half and
// unit instead of per group.  The staged activations of a unit are 512 dense bytes, read
// with one 128-bit load per lane into the register set of the lane's own group; the sets of
// the other groups stay zero for the whole kernel.  Lanes that share an output row add their
// partial sums with two shuffles in the epilogue.
template <bool kScaleF16>
struct UnitScale {
  typename std::conditional<kScaleF16, uint32_t, uint2>::type v;  // rows g, g+8 of the lane's own group
};

template <typename XT, bool kScaleF16, int kG, int kD>
__global__ void __launch_bounds__(kWarps * 32)
qgemv_i4_gp_kernel(const GemvParams p) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;  // chunk bytes
  constexpr int kCpg = 8 / kG;                 // MMA columns per group
  constexpr int kCU = kG / 2;                  // chunks per unit
  constexpr int kUnits = kD / kCU;         // ring entries
  constexpr int kCorrStride = kHasLo ? kCpg / 2 : kCpg;  // activation rows a group's columns hold
  constexpr int kAcc = kHasLo ? 2 : 4;
  constexpr int kCorr = kHasLo ? 1 : 2;
  constexpr uint32_t kTileRowsCta = kWarps * 16;
  constexpr uint32_t kXsStride = kCpg * 64;    // staged bytes per group
  static_assert(kG == 2 || kG == 4, "units of two or four groups");
  static_assert(kD % kCU == 0, "the ring holds whole units");

  extern __shared__ __align__(16) uint8_t smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;

  pdl_launch_dependents();

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
  const uint32_t cbeg = min(split * p.chunks_per_split, chunks_per_row);
  const uint32_t cend = min(cbeg + p.chunks_per_split, chunks_per_row);
  const uint32_t nch = cend - cbeg;  // a whole number of units (the host guarantees it)

  const uint32_t active_cols = kHasLo ? 2 * p.m : p.m;
  uint8_t* xs = smem;
  float* corr = reinterpret_cast<float*>(smem + 2 * p.slab_chunks * kXsStride);

  // the group (inside a unit) and the activation row(s) this lane's two C columns belong to
  const uint32_t jl = (2u * t) / kCpg;
  const uint32_t tl = t % (kCpg / 2);
  // the group whose activations this lane feeds the MMAs with (B operand: column g)
  const uint32_t jb = g / kCpg;
  const bool col_live = (g % kCpg) < active_cols;

  const uint8_t* next = w_base + (static_cast<size_t>(row_block) * chunks_per_row + cbeg) * kCB + lane * 16;
  const uint32_t scale_off = (jl >> 1) * kCB + kChunkWeightBytes - lane * 16 + g * (4 * kScaleBytes) +
                             (jl & 1u) * (2 * kScaleBytes);

  uint4 ring_w[kUnits][kCU];
  UnitScale<kScaleF16> ring_s[kUnits];
  auto fetch = [&](const int u, const uint8_t* src) {
#pragma unroll
    for (int c = 0; c < kCU; ++c) ring_w[u][c] = ldg_stream_v4(src + c * kCB);
    if constexpr (kScaleF16) ring_s[u].v = ldg_stream_u32(src + scale_off);
    else ring_s[u].v = ldg_stream_v2(src + scale_off);
  };
#pragma unroll
  for (int u = 0; u < kUnits; ++u) {
#pragma unroll
    for (int c = 0; c < kCU; ++c) ring_w[u][c] = make_uint4(0, 0, 0, 0);
    if constexpr (kScaleF16) ring_s[u].v = 0u;
    else ring_s[u].v = make_uint2(0, 0);
    if (active && static_cast<uint32_t>(u * kCU) < nch) fetch(u, next + u * (kCU * kCB));
  }
  next += kD * kCB;

  pdl_wait_prior_grid();
  // the epoch of this exchange: written by the previous fused launch, which has finished now
  const unsigned int epoch = p.fcomm != nullptr ? *reinterpret_cast<volatile unsigned int*>(p.fcomm->epoch) + 1u : 0u;

  float acc[kAcc];
#pragma unroll
  for (int j = 0; j < kAcc; ++j) acc[j] = 0.0f;
  constexpr uint32_t kMask0 = 0x000F000Fu, kMask1 = 0x00F000F0u;

  uint4 bset[kG];
  bool load_b[kG];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    bset[j] = make_uint4(0, 0, 0, 0);
    load_b[j] = col_live && jb == static_cast<uint32_t>(j);
  }
  float cterm[kCorr], cinv[kCorr];  // {-8 sum x, 2^-e} of the lane's own group and activation rows
  bool load_c[kCorr];
#pragma unroll
  for (int j = 0; j < kCorr; ++j) {
    cterm[j] = 0.0f;
    cinv[j] = 0.0f;
    load_c[j] = (kHasLo ? tl : 2 * tl + j) < p.m;
  }
  const uint32_t xs_lane = static_cast<uint32_t>(__cvta_generic_to_shared(xs)) + lane * 16;
  const uint32_t corr_lane = static_cast<uint32_t>(__cvta_generic_to_shared(corr)) +
                             (jl * kCorrStride + (kHasLo ? tl : 2 * tl)) * 8;

  auto process = [&](const int u, uint32_t xs_addr, uint32_t corr_addr, bool refill) {
#pragma unroll
    for (int j = 0; j < kG; ++j) lds_v4_if(bset[j], xs_addr, load_b[j]);
#pragma unroll
    for (int j = 0; j < kCorr; ++j) lds_v2f_if(cterm[j], cinv[j], corr_addr + j * 8, load_c[j]);
    float cf[4];
#pragma unroll
    for (int j = 0; j < kG; ++j) {
      const uint4 wq = ring_w[u][j >> 1];
      const uint32_t wa = (j & 1) ? wq.z : wq.x;  // row g
      const uint32_t wb = (j & 1) ? wq.w : wq.y;  // row g + 8
      const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
      const uint32_t a0[4] = {wa & kMask0, wb & kMask0, wa & kMask1, wb & kMask1};
      const uint32_t a1[4] = {wa8 & kMask0, wb8 & kMask0, wa8 & kMask1, wb8 & kMask1};
      if (j == 0) mma_f16_zero(cf, a0, bset[j].x, bset[j].y);
      else mma_f16(cf, a0, bset[j].x, bset[j].y);
      mma_f16(cf, a1, bset[j].z, bset[j].w);
    }
    float2 s;  // .x = row g, .y = row g + 8, the lane's own group
    if constexpr (kScaleF16) s = __half22float2(*reinterpret_cast<const __half2*>(&ring_s[u].v));
    else s = make_float2(__uint_as_float(ring_s[u].v.x), __uint_as_float(ring_s[u].v.y));
    if constexpr (kHasLo) {
      acc[0] = fmaf(s.x, fmaf(cf[0] + cf[1], cinv[0], cterm[0]), acc[0]);
      acc[1] = fmaf(s.y, fmaf(cf[2] + cf[3], cinv[0], cterm[0]), acc[1]);
    } else {
      acc[0] = fmaf(s.x, fmaf(cf[0], cinv[0], cterm[0]), acc[0]);
      acc[1] = fmaf(s.x, fmaf(cf[1], cinv[1], cterm[1]), acc[1]);
      acc[2] = fmaf(s.y, fmaf(cf[2], cinv[0], cterm[0]), acc[2]);
      acc[3] = fmaf(s.y, fmaf(cf[3], cinv[1], cterm[1]), acc[3]);
    }
    if (refill && active) fetch(u, next + u * (kCU * kCB));
  };

  const XT* x = static_cast<const XT*>(p.x);
  for (uint32_t done = 0; done < nch;) {
    const uint32_t slab_n = min(p.slab_chunks, nch - done);
    if (done != 0) __syncthreads();
    stage_x<XT, kHasLo, kCorrStride>(x, p.m, p.k, 2 * (cbeg + done), 2 * slab_n, xs, kXsStride, corr);
    __syncthreads();
    uint32_t xs_addr = xs_lane, corr_addr = corr_lane;
    uint32_t i = 0;
    for (; i + kD <= slab_n; i += kD) {
#pragma unroll
      for (int u = 0; u < kUnits; ++u) {
        process(u, xs_addr, corr_addr, done + i + u * kCU + kD < nch);
        xs_addr += 512;
        corr_addr += kG * kCorrStride * 8;
      }
      next += kD * kCB;
    }
#pragma unroll
    for (int u = 0; u < kUnits - 1; ++u) {  // the last, short round of the split
      if (i + u * kCU < slab_n) {
        process(u, xs_addr, corr_addr, false);
        xs_addr += 512;
        corr_addr += kG * kCorrStride * 8;
      }
    }
    done += slab_n;
  }

  // ---- epilogue: lanes whose C columns belong to different groups hold partial sums of the
  // same outputs; add them (fixed order), then the lanes of group 0 own the result.
#pragma unroll
  for (int j = 0; j < kAcc; ++j) {
    if constexpr (kG == 4) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 1);
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 2);
  }
  float* red = reinterpret_cast<float*>(smem);  // [m][kTileRowsCta], aliases the x slab
  const bool fused = p.fcomm != nullptr;
  if (p.splits > 1 || fused) __syncthreads();
  if (active && jl == 0) {
    const uint32_t row_a = row_block * 16u + g;
    const uint32_t tr_a = warp * 16u + g;
#pragma unroll
    for (int j = 0; j < (kHasLo ? 1 : 2); ++j) {
      const uint32_t mm = kHasLo ? tl : 2 * tl + j;
      if (mm >= p.m) continue;
      const float va = acc[kHasLo ? 0 : j];
      const float vb = acc[kHasLo ? 1 : 2 + j];
      if (p.splits == 1 && !fused) {
        out[static_cast<size_t>(mm) * n + row_a] = fmaf(va, kUnscale, bias[row_a]);
        out[static_cast<size_t>(mm) * n + row_a + 8] = fmaf(vb, kUnscale, bias[row_a + 8]);
      } else {
        red[mm * kTileRowsCta + tr_a] = va;
        red[mm * kTileRowsCta + tr_a + 8] = vb;
      }
    }
  }
  if (fused) {
    reduce_exchange_store(p, red, kTileRowsCta, tile, split, n, out, bias, epoch);
    return;
  }
  if (p.splits == 1) return;
  cluster_reduce_store(p, red, kTileRowsCta, tile, split, n, out, bias);
}

template <typename XT, int kCols>
uint32_t group_smem_bytes(uint32_t m) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  return (kHasLo ? 2 * m : m) * 64 + (kHasLo ? kCols / 2 : kCols) * 8;  // staged halves + {corr, 2^-e} pairs
}

template <typename XT, bool kScaleF16, int kCols, int kRB>
cudaError_t launch_typed(const LaunchEnv& env, GemvParams& p, int count, const LinearTarget* targets) {
  auto kernel = qgemv_i4_kernel<XT, kScaleF16, kCols, kRB>;
  static PerDevice<bool> configured_on;
  bool* configured = configured_on.slot();
  if (configured == nullptr) return cudaErrorInvalidDevice;
  if (!*configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return e;
    *configured = true;
  }
  constexpr uint32_t kTileRowsCta = kWarps * kRB * 16;
  uint32_t tiles = 0;
  for (int i = 0; i < count; ++i) {
    p.tile_begin[i] = tiles;
    tiles += (targets[i].w->n + kTileRowsCta - 1) / kTileRowsCta;
  }
  for (int i = count; i <= kMaxMulti; ++i) p.tile_begin[i] = tiles;

  const uint32_t chunks_per_row = p.k / kChunkK;

  // Split K over a cluster until the grid fills the machine (about four CTAs per SM);
  // a pure function of the shape, never autotuned.
  const uint32_t want_ctas = static_cast<uint32_t>(env.sm_count) * kWantCtasPerSm;
  uint32_t splits = 1;
  while (splits < static_cast<uint32_t>(kMaxCluster) && tiles * splits < want_ctas &&
         splits * 2 <= chunks_per_row)
    splits *= 2;
  p.splits = splits;
  p.chunks_per_split = (chunks_per_row + splits - 1) / splits;
  // Activations are staged at most ~32 KB at a time; a slab that is not the last one of
  // its split must be a whole number of ring rounds.
  const uint32_t per_chunk = 2 * group_smem_bytes<XT, kCols>(p.m);
  uint32_t slab_cap = std::max<uint32_t>(kDepth, (32768u / per_chunk) / kDepth * kDepth);
  p.slab_chunks = std::max<uint32_t>(1u, std::min(p.chunks_per_split, slab_cap));

  const size_t slab_bytes = static_cast<size_t>(p.slab_chunks) * per_chunk;
  const size_t red_bytes = splits > 1 ? static_cast<size_t>(p.m) * kTileRowsCta * sizeof(float) : 0;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, splits, 1);
  cfg.blockDim = dim3(kWarps * 32, 1, 1);
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

// How many CTAs of a launch configuration fit on the device at the same time (0 when the
// query fails, which callers treat as "does not fit").  The decision the fused exchange
// depends on: its CTAs wait for their twins on the other GPUs, so the whole grid has to be
// resident in one wave.
struct ResidencyKey {
  const void* kernel;
  int device;
  size_t smem;
  uint32_t splits;
  uint32_t ctas;
};
uint32_t resident_ctas(const void* kernel, int device, const cudaLaunchConfig_t& cfg, uint32_t splits, int sm_count) {
  static ResidencyKey cache[64];
  static int cached = 0;
  for (int i = 0; i < cached; ++i)
    if (cache[i].kernel == kernel && cache[i].device == device && cache[i].smem == cfg.dynamicSmemBytes &&
        cache[i].splits == splits)
      return cache[i].ctas;
  uint32_t ctas = 0;
  if (splits > 1) {
    cudaLaunchConfig_t probe = cfg;
    cudaLaunchAttribute cluster;
    cluster.id = cudaLaunchAttributeClusterDimension;
    cluster.val.clusterDim.x = 1;
    cluster.val.clusterDim.y = splits;
    cluster.val.clusterDim.z = 1;
    probe.attrs = &cluster;
    probe.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &probe) == cudaSuccess && clusters > 0)
      ctas = static_cast<uint32_t>(clusters) * splits;
  } else {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, static_cast<int>(cfg.blockDim.x),
                                                      cfg.dynamicSmemBytes) == cudaSuccess && per_sm > 0)
      ctas = static_cast<uint32_t>(per_sm) * static_cast<uint32_t>(sm_count);
  }
  (void)cudaGetLastError();
  if (cached < 64) cache[cached++] = ResidencyKey{kernel, device, cfg.dynamicSmemBytes, splits, ctas};
  return ctas;
}

template <typename XT, bool kScaleF16, int kG, int kD>
cudaError_t launch_typed_gp_depth(const LaunchEnv& env, GemvParams& p, int count, const LinearTarget* targets,
                                  bool probe_only, uint32_t* ctas_out, uint32_t* capacity_out) {
  auto kernel = qgemv_i4_gp_kernel<XT, kScaleF16, kG, kD>;
  struct Setup { bool done; uint32_t max_cluster; };
  static PerDevice<Setup> setup_on;
  Setup* setup = setup_on.slot();
  if (setup == nullptr) return cudaErrorInvalidDevice;
  uint32_t& max_cluster = setup->max_cluster;
  if (!setup->done) {
    max_cluster = kMaxCluster;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return e;
    // few row tiles and a long k (8960 -> 1536): sixteen splits, the largest cluster the device
    // takes with this opt-in, halve each CTA's share again
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) max_cluster = 16;
    else (void)cudaGetLastError();
    setup->done = true;
  }
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kCpg = 8 / kG, kCU = kG / 2;
  constexpr uint32_t kCorrStride = kHasLo ? kCpg / 2 : kCpg;
  constexpr uint32_t kTileRowsCta = kWarps * 16;
  uint32_t tiles = 0;
  for (int i = 0; i < count; ++i) {
    p.tile_begin[i] = tiles;
    tiles += (targets[i].w->n + kTileRowsCta - 1) / kTileRowsCta;
  }
  for (int i = count; i <= kMaxMulti; ++i) p.tile_begin[i] = tiles;

  const uint32_t units_per_row = p.k / kChunkK / kCU;  // the caller checked divisibility
  const uint32_t want_ctas = static_cast<uint32_t>(env.sm_count) * kWantCtasPerSm;
  uint32_t splits = 1;
  // ... and, once every SM has a CTA, as long as a split keeps at least six chunks of k: below that
  // a CTA's fixed cost (staging, cluster reduction) outweighs its share of the stream
  // (1536 -> 8960: 5.3 us with four splits of six chunks, 7.9 us with eight of at most four).
  constexpr uint32_t kMinUnits = 6 / kCU;
  const uint32_t split_limit = env.fused != nullptr ? static_cast<uint32_t>(kMaxCluster) : max_cluster;
  while (splits < split_limit && tiles * splits < want_ctas && splits * 2 <= units_per_row &&
         (tiles * splits < static_cast<uint32_t>(env.sm_count) || splits * 2 * kMinUnits <= units_per_row))
    splits *= 2;
  p.splits = splits;
  p.chunks_per_split = (units_per_row + splits - 1) / splits * kCU;
  const uint32_t per_chunk = 2 * (kCpg * 64 + kCorrStride * 8);
  const uint32_t slab_cap = std::max<uint32_t>(kD, (32768u / per_chunk) / kD * kD);
  p.slab_chunks = std::max<uint32_t>(kCU, std::min(p.chunks_per_split, slab_cap));

  const size_t slab_bytes = static_cast<size_t>(p.slab_chunks) * per_chunk;
  p.fcomm = env.fused;
  const size_t red_bytes = (splits > 1 || env.fused != nullptr) ? static_cast<size_t>(p.m) * kTileRowsCta * sizeof(float) : 0;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, splits, 1);
  cfg.blockDim = dim3(kWarps * 32, 1, 1);
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
  if (ctas_out) *ctas_out = tiles * splits;
  if (capacity_out) {
    // CTAs of THIS launch that can be resident at once: asked with the launch's own dynamic
    // shared memory and, when K is split, its cluster shape (clusters co-schedule fewer CTAs
    // than the per-SM limit suggests).  Cached per (device, shared memory, splits).
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    *capacity_out = resident_ctas(reinterpret_cast<const void*>(kernel), device, cfg, splits, env.sm_count);
  }
  if (probe_only) return cudaSuccess;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

// A ring twice as deep keeps every byte of a small matrix in flight at once, but costs
// registers: worth it only while the whole grid is still resident in one wave.  The fused
// exchange NEEDS one wave (its CTAs wait for their twins on the other GPUs): when the grid
// does not fit, the caller gets cudaErrorNotSupported and runs the exchange separately.
template <typename XT, bool kScaleF16, int kG>
cudaError_t launch_typed_gp(const LaunchEnv& env, GemvParams& p, int count, const LinearTarget* targets) {
  uint32_t ctas = 0, capacity = 0;
  cudaError_t e = launch_typed_gp_depth<XT, kScaleF16, kG, 2 * kDepth>(env, p, count, targets, true, &ctas, &capacity);
  if (e != cudaSuccess) return e;
  if (env.fused != nullptr && (count != 1 || ctas > kFusedMaxCtas ||
                               static_cast<uint64_t>(p.m) * targets[0].w->n * 8u > kFusedSlotBytes))
    return cudaErrorNotSupported;
  if (ctas <= capacity)
    return launch_typed_gp_depth<XT, kScaleF16, kG, 2 * kDepth>(env, p, count, targets, false, nullptr, nullptr);
  if (env.fused != nullptr) {
    e = launch_typed_gp_depth<XT, kScaleF16, kG, kDepth>(env, p, count, targets, true, &ctas, &capacity);
    if (e != cudaSuccess) return e;
    if (ctas > capacity) return cudaErrorNotSupported;
  }
  return launch_typed_gp_depth<XT, kScaleF16, kG, kDepth>(env, p, count, targets, false, nullptr, nullptr);
}

// Converts the whole activation block to the staged layout ONCE per launch, into global
// scratch.  With many activation rows the conversion is as much work as a CTA's share of the
// matmul, and every CTA would repeat it for its k range; this way a CTA only copies bytes.
// The wide kernel pre-scales each activation ROW by one power of two (a per-group factor would
// have to multiply every C value of every group; a per-row one leaves the inner loop alone and
// is applied once in the epilogue): scale[row] = 2^e, inv[row] = 2^-e (kq_gemv_core.cuh:
// pow2_prescale).
// One launch: CTA (row, slice) finds the largest magnitude of its activation row (every slice
// of a row repeats that pass: a row is at most a few tens of KB, read from L2), derives the
// row's power-of-two scale, and converts its slice of the row's 32-k groups.  Slice 0 also
// publishes scale[row] and inv[row] = 2^-e for the matmul's epilogue.
template <typename XT, int kTiles>
__global__ void __launch_bounds__(256)
stage_x_global_kernel(const XT* __restrict__ x, uint32_t m, uint32_t k, uint8_t* xs, float* corr, float* scale_out,
                      float* inv_out, const float* __restrict__ norm_weight, float norm_eps) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kLoOffset = kTiles * 512u;
  constexpr uint32_t kXsStride = kLoOffset * (kHasLo ? 2u : 1u);
  const uint32_t row = blockIdx.x, slice = blockIdx.y, slices = gridDim.y;
  const XT* xr = x + static_cast<size_t>(row) * k;
  __shared__ float part[8];
  __shared__ float scale_s[16];
  __shared__ float r_inv_s;
  // With an rms_norm in front (packages/runtime/src/kernels/rms-norm.ts:60-90) what is staged is
  // (x * rsqrt(mean(x^2) + eps)) * weight: one more pass over the row for the sum of squares,
  // added in a fixed order (thread-strided, shuffle tree, warps in order).
  float r_inv = 1.0f;
  if (norm_weight != nullptr) {
    float sq = 0.0f;
    for (uint32_t i = threadIdx.x * 8; i < k; i += blockDim.x * 8) {
      float v[8];
      load_x8<XT>(xr + i, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) sq = fmaf(v[e], v[e], sq);
    }
    sq = warp_sum(sq);
    if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.0f;
      for (int w = 0; w < 8; ++w) total += part[w];
      r_inv_s = rsqrtf(total * (1.0f / static_cast<float>(k)) + norm_eps);
    }
    __syncthreads();
    r_inv = r_inv_s;
  }
  auto load_row8 = [&](uint32_t i, float (&v)[8]) {
    load_x8<XT>(xr + i, v);
    if (norm_weight != nullptr) {
      const float4 w0 = __ldg(reinterpret_cast<const float4*>(norm_weight + i));
      const float4 w1 = __ldg(reinterpret_cast<const float4*>(norm_weight + i + 4));
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(__fmul_rn(v[e], r_inv), wv[e]);
    }
  };
  float amax = 0.0f;
  for (uint32_t i = threadIdx.x * 8; i < k; i += blockDim.x * 8) {  // k is a multiple of 64
    float v[8];
    load_row8(i, v);
    amax = fmaxf(amax, absmax8(v));
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, part[w]);
    const Pow2 ps = pow2_prescale(amax);
    scale_s[row] = ps.scale;
    if (slice == 0) {
      scale_out[row] = ps.scale;
      inv_out[row] = ps.inv;
    }
  }
  __syncthreads();
  const uint32_t groups = k / 32, per_slice = (groups + slices - 1) / slices;
  const uint32_t g0 = min(slice * per_slice, groups), g1 = min(g0 + per_slice, groups);
  const uint32_t items = (g1 - g0) * 4, items_padded = (items + 31u) & ~31u;  // whole warps run the shuffles
  for (uint32_t item = threadIdx.x; item < items_padded; item += blockDim.x) {
    const bool valid = item < items;
    const uint32_t lg = g0 + (item >> 2), q = item & 3u;
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (valid) load_row8((lg << 5) + (q << 3), v);
    stage_octet<kHasLo, kTiles * 8, false>(v, valid, q, row, lg, xs, kXsStride, corr, kHasLo ? kLoOffset : 0u, scale_s);
  }
}

// ---- wide variant: more than 4 MMA columns (3 to 16 activation rows) -------------------
// Column c of tile j is activation row 8 j + c for every input type.  The hi and lo parts of
// an f32 / bf16 activation are two B operands that accumulate into the SAME C tile (two more
// MMAs per group instead of twice the columns), and the "-8 sum x" term enters as the C
// operand of the group's first MMA, so all that is left per group and C value is one FFMA
// with the group scale.  Two row blocks per warp share every shared-memory load.
template <typename XT, bool kScaleF16, int kTiles, int kRB, int kD>
__global__ void __launch_bounds__(kWarps * 32)
qgemv_i4_wide_kernel(const GemvParams p) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;  // chunk bytes
  constexpr int kCols = kTiles * 8;
  constexpr uint32_t kLoOffset = kTiles * 512u;
  constexpr uint32_t kXsStride = kLoOffset * (kHasLo ? 2u : 1u);
  constexpr uint32_t kTileRowsCta = kWarps * kRB * 16;

  extern __shared__ __align__(16) uint8_t smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;

  pdl_launch_dependents();

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
  const uint32_t row_block0 = (tile * kWarps + warp) * kRB;

  const uint32_t chunks_per_row = p.k / kChunkK;
  const uint32_t split = blockIdx.y;
  const uint32_t cbeg = min(split * p.chunks_per_split, chunks_per_row);
  const uint32_t cend = min(cbeg + p.chunks_per_split, chunks_per_row);
  const uint32_t nch = cend - cbeg;

  uint8_t* xs = smem;
  float* corr = reinterpret_cast<float*>(smem + 2 * p.slab_chunks * kXsStride);

  bool active[kRB];
  const uint8_t* next[kRB];
#pragma unroll
  for (int r = 0; r < kRB; ++r) {
    active[r] = (row_block0 + r) * 16u < n;
    next[r] = w_base + (static_cast<size_t>(row_block0 + r) * chunks_per_row + cbeg) * kCB + lane * 16;
  }
  const uint32_t scale_off = kChunkWeightBytes - lane * 16 + g * (4 * kScaleBytes);

  ChunkRegs<kScaleF16> ring[kD][kRB];
  auto fetch = [&](ChunkRegs<kScaleF16>& dst, const uint8_t* src) {
    dst.w = ldg_stream_v4(src);
    if constexpr (kScaleF16) dst.s = ldg_stream_v2(src + scale_off);
    else dst.s = ldg_stream_v4(src + scale_off);
  };
#pragma unroll
  for (int d = 0; d < kD; ++d)
#pragma unroll
    for (int r = 0; r < kRB; ++r) {
      ring[d][r].w = make_uint4(0, 0, 0, 0);
      if constexpr (kScaleF16) ring[d][r].s = make_uint2(0, 0);
      else ring[d][r].s = make_uint4(0, 0, 0, 0);
      if (active[r] && static_cast<uint32_t>(d) < nch) fetch(ring[d][r], next[r] + d * kCB);
    }
#pragma unroll
  for (int r = 0; r < kRB; ++r) next[r] += kD * kCB;

  pdl_wait_prior_grid();

  float acc[kRB][kTiles][4];
#pragma unroll
  for (int r = 0; r < kRB; ++r)
#pragma unroll
    for (int i = 0; i < kTiles; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[r][i][j] = 0.0f;

  constexpr uint32_t kMask0 = 0x000F000Fu, kMask1 = 0x00F000F0u;

  uint4 bhi[kTiles], blo[kTiles];
  float cterm[kTiles][2];
  bool load_b[kTiles], load_c[kTiles][2];
#pragma unroll
  for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
    bhi[tile_m] = make_uint4(0, 0, 0, 0);
    blo[tile_m] = make_uint4(0, 0, 0, 0);
    load_b[tile_m] = tile_m * 8 + g < p.m;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      cterm[tile_m][j] = 0.0f;
      load_c[tile_m][j] = tile_m * 8 + 2 * t + j < p.m;
    }
  }
  const uint32_t xs_lane = static_cast<uint32_t>(__cvta_generic_to_shared(xs)) + lane * 16;
  const uint32_t corr_lane = static_cast<uint32_t>(__cvta_generic_to_shared(corr)) + 2 * t * 4;

  auto process = [&](const int d, uint32_t xs_addr, uint32_t corr_addr, bool refill) {
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
#pragma unroll
      for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
        lds_v4_if(bhi[tile_m], xs_addr + jj * kXsStride + tile_m * 512, load_b[tile_m]);
        if constexpr (kHasLo) lds_v4_if(blo[tile_m], xs_addr + jj * kXsStride + kLoOffset + tile_m * 512, load_b[tile_m]);
#pragma unroll
        for (int j = 0; j < 2; ++j)
          lds_f32_if(cterm[tile_m][j], corr_addr + (jj * kCols + tile_m * 8 + j) * 4, load_c[tile_m][j]);
      }
#pragma unroll
      for (int r = 0; r < kRB; ++r) {
        const uint32_t wa = jj ? ring[d][r].w.z : ring[d][r].w.x;  // row g
        const uint32_t wb = jj ? ring[d][r].w.w : ring[d][r].w.y;  // row g + 8
        const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
        const uint32_t a0[4] = {wa & kMask0, wb & kMask0, wa & kMask1, wb & kMask1};
        const uint32_t a1[4] = {wa8 & kMask0, wb8 & kMask0, wa8 & kMask1, wb8 & kMask1};
        float2 s;  // .x = row g, .y = row g + 8
        if constexpr (kScaleF16) {
          s = __half22float2(*reinterpret_cast<const __half2*>(jj ? &ring[d][r].s.y : &ring[d][r].s.x));
        } else {
          s = jj ? make_float2(__uint_as_float(ring[d][r].s.z), __uint_as_float(ring[d][r].s.w))
                 : make_float2(__uint_as_float(ring[d][r].s.x), __uint_as_float(ring[d][r].s.y));
        }
#pragma unroll
        for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
          float cf[4];
          mma_f16_init(cf, a0, bhi[tile_m].x, bhi[tile_m].y, cterm[tile_m][0], cterm[tile_m][1]);
          mma_f16(cf, a1, bhi[tile_m].z, bhi[tile_m].w);
          if constexpr (kHasLo) {
            mma_f16(cf, a0, blo[tile_m].x, blo[tile_m].y);
            mma_f16(cf, a1, blo[tile_m].z, blo[tile_m].w);
          }
          acc[r][tile_m][0] = fmaf(s.x, cf[0], acc[r][tile_m][0]);
          acc[r][tile_m][1] = fmaf(s.x, cf[1], acc[r][tile_m][1]);
          acc[r][tile_m][2] = fmaf(s.y, cf[2], acc[r][tile_m][2]);
          acc[r][tile_m][3] = fmaf(s.y, cf[3], acc[r][tile_m][3]);
        }
      }
    }
    if (refill) {
#pragma unroll
      for (int r = 0; r < kRB; ++r)
        if (active[r]) fetch(ring[d][r], next[r] + d * kCB);
    }
  };

  for (uint32_t done = 0; done < nch;) {
    const uint32_t slab_n = min(p.slab_chunks, nch - done);
    if (done != 0) __syncthreads();
    {  // the activations were converted once per launch by stage_x_global_kernel: copy bytes
      const uint32_t first_group = 2 * (cbeg + done);
      const uint4* src = reinterpret_cast<const uint4*>(p.staged_xs + static_cast<size_t>(first_group) * kXsStride);
      uint4* dst = reinterpret_cast<uint4*>(xs);
      const uint32_t n16 = 2 * slab_n * (kXsStride / 16);
      for (uint32_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = __ldg(src + i);
      const float4* csrc = reinterpret_cast<const float4*>(p.staged_corr + static_cast<size_t>(first_group) * kCols);
      float4* cdst = reinterpret_cast<float4*>(corr);
      const uint32_t c16 = 2 * slab_n * (kCols / 4);
      for (uint32_t i = threadIdx.x; i < c16; i += blockDim.x) cdst[i] = __ldg(csrc + i);
    }
    __syncthreads();
    uint32_t xs_addr = xs_lane, corr_addr = corr_lane;
    uint32_t i = 0;
    for (; i + kD <= slab_n; i += kD) {
#pragma unroll
      for (int d = 0; d < kD; ++d) {
        process(d, xs_addr, corr_addr, done + i + d + kD < nch);
        xs_addr += 2 * kXsStride;
        corr_addr += 2 * kCols * 4;
      }
#pragma unroll
      for (int r = 0; r < kRB; ++r) next[r] += kD * kCB;
    }
#pragma unroll
    for (int d = 0; d < kD - 1; ++d) {
      if (i + d < slab_n) {
        process(d, xs_addr, corr_addr, false);
        xs_addr += 2 * kXsStride;
        corr_addr += 2 * kCols * 4;
      }
    }
    done += slab_n;
  }

  // lane owns rows g, g+8 of each block and activation rows 8 tile + 2t, 2t+1
  float* red = reinterpret_cast<float*>(smem);
  if (p.splits > 1) __syncthreads();
#pragma unroll
  for (int r = 0; r < kRB; ++r) {
    if (!active[r]) continue;
    const uint32_t row_a = (row_block0 + r) * 16u + g;
    const uint32_t tr_a = (warp * kRB + r) * 16u + g;
    float bias_a = 0.0f, bias_b = 0.0f;
    if (p.splits == 1) {
      bias_a = bias[row_a];
      bias_b = bias[row_a + 8];
    }
#pragma unroll
    for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t mm = tile_m * 8 + 2 * t + j;
        if (mm >= p.m) continue;
        const float inv = __ldg(p.staged_inv + mm);  // undo the row's power-of-two pre-scale (exact)
        const float va = acc[r][tile_m][j] * inv, vb = acc[r][tile_m][2 + j] * inv;
        if (p.splits == 1) {
          float oa = fmaf(va, kUnscale, bias_a), ob = fmaf(vb, kUnscale, bias_b);
          if (p.residual != nullptr) {
            oa = __fadd_rn(oa, p.residual[static_cast<size_t>(mm) * n + row_a]);
            ob = __fadd_rn(ob, p.residual[static_cast<size_t>(mm) * n + row_a + 8]);
          }
          out[static_cast<size_t>(mm) * n + row_a] = oa;
          out[static_cast<size_t>(mm) * n + row_a + 8] = ob;
        } else {
          red[mm * kTileRowsCta + tr_a] = va;
          red[mm * kTileRowsCta + tr_a + 8] = vb;
        }
      }
    }
  }
  if (p.splits == 1) return;
  cluster_reduce_store(p, red, kTileRowsCta, tile, split, n, out, bias);
}

template <typename XT, bool kScaleF16, int kTiles, int kRB, int kD>
cudaError_t launch_typed_wide(const LaunchEnv& env, GemvParams& p, int count, const LinearTarget* targets,
                              int* extra_launches) {
  auto kernel = qgemv_i4_wide_kernel<XT, kScaleF16, kTiles, kRB, kD>;
  static PerDevice<bool> configured_on;
  bool* configured = configured_on.slot();
  if (configured == nullptr) return cudaErrorInvalidDevice;
  if (!*configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) return e;
    *configured = true;
  }
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kTileRowsCta = kWarps * kRB * 16;
  uint32_t tiles = 0;
  for (int i = 0; i < count; ++i) {
    p.tile_begin[i] = tiles;
    tiles += (targets[i].w->n + kTileRowsCta - 1) / kTileRowsCta;
  }
  for (int i = count; i <= kMaxMulti; ++i) p.tile_begin[i] = tiles;
  const uint32_t chunks_per_row = p.k / kChunkK;
  const uint32_t want_ctas = static_cast<uint32_t>(env.sm_count) * kWantCtasPerSm;
  uint32_t splits = 1;
  while (splits < static_cast<uint32_t>(kMaxCluster) && tiles * splits < want_ctas && splits * 2 <= chunks_per_row)
    splits *= 2;
  p.splits = splits;
  p.chunks_per_split = (chunks_per_row + splits - 1) / splits;
  const uint32_t per_chunk = 2 * (kTiles * 512u * (kHasLo ? 2u : 1u) + kTiles * 8u * 4u);
  const uint32_t slab_cap = std::max<uint32_t>(kD, (kWideSlabBytes * kTiles / per_chunk) / kD * kD);
  p.slab_chunks = std::max<uint32_t>(1u, std::min(p.chunks_per_split, slab_cap));
  const size_t slab_bytes = static_cast<size_t>(p.slab_chunks) * per_chunk;
  const size_t red_bytes = splits > 1 ? static_cast<size_t>(p.m) * kTileRowsCta * sizeof(float) : 0;

  // Convert the activations once per launch, into the context's scratch: row scales, staged
  // halves and the "-8 sum x" terms, one pre-kernel.
  const uint32_t groups = p.k / 32;
  const size_t xs_total = static_cast<size_t>(groups) * (kTiles * 512u * (kHasLo ? 2u : 1u));
  const size_t corr_total = static_cast<size_t>(groups) * kTiles * 8u * sizeof(float);
  const size_t scale_total = 2 * 16 * sizeof(float);
  if (env.workspace == nullptr || xs_total + corr_total + scale_total > env.workspace_bytes)
    return cudaErrorMemoryAllocation;  // the context's workspace is too small for this k
  {
    uint8_t* ws = static_cast<uint8_t*>(env.workspace);
    float* corr_ws = reinterpret_cast<float*>(ws + xs_total);
    float* scale_ws = reinterpret_cast<float*>(ws + xs_total + corr_total);
    const uint32_t slices = std::max(1u, std::min(8u, groups / 32));  // at least 32 groups per CTA
    stage_x_global_kernel<XT, kTiles><<<dim3(p.m, slices), 256, 0, env.stream>>>(
        static_cast<const XT*>(p.x), p.m, p.k, ws, corr_ws, scale_ws, scale_ws + 16, env.norm_weight, env.norm_eps);
    p.residual = env.residual;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    p.staged_xs = ws;
    p.staged_corr = corr_ws;
    p.staged_inv = scale_ws + 16;
    if (extra_launches) *extra_launches += 1;
  }

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, splits, 1);
  cfg.blockDim = dim3(kWarps * 32, 1, 1);
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

// Columns of the MMA tile an activation row needs: 1 for binary16 input, 2 (hi, lo)
// for f32 / bf16 input.  One row block per warp while a single MMA tile holds every
// column; two (sharing the B fragments) beyond that, where shared-memory bandwidth
// would otherwise bound the kernel.
template <typename XT>
cudaError_t launch_x(const LaunchEnv& env, GemvParams& p, int count, const LinearTarget* t, bool f16s, int* extra) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  const uint32_t cols = kHasLo ? 2 * p.m : p.m;
  // Few columns: pack several scale groups into one MMA tile (four groups need an even
  // number of 64-k chunks per row).
  if (cols <= 2 && (p.k / kChunkK) % 2 == 0)
    return f16s ? launch_typed_gp<XT, true, 4>(env, p, count, t) : launch_typed_gp<XT, false, 4>(env, p, count, t);
  if (cols <= 4)
    return f16s ? launch_typed_gp<XT, true, 2>(env, p, count, t) : launch_typed_gp<XT, false, 2>(env, p, count, t);
  if (env.fused != nullptr) return cudaErrorNotSupported;  // only the group-packed kernel exchanges in its epilogue
  if (kHasLo && p.m <= 4)  // three or four f32 / bf16 rows: hi and lo in adjacent columns of one tile
    return f16s ? launch_typed<XT, true, 8, 1>(env, p, count, t) : launch_typed<XT, false, 8, 1>(env, p, count, t);
  // Five or more rows.  Two row blocks per warp (sharing the activation loads) pay off when a
  // row block costs many MMAs (hi + lo parts, or two column tiles) and the matrix has rows to
  // spare; otherwise one row block per warp and a deeper ring keep more CTAs in flight.  A pure
  // function of the shape.
  uint32_t row_blocks = 0;
  for (int i = 0; i < count; ++i) row_blocks += t[i].w->n / 16;
  const bool heavy = kHasLo || p.m > 8;
  const bool pair = heavy && row_blocks >= 1024;
  if (p.m <= 8) {
    if (pair)
      return f16s ? launch_typed_wide<XT, true, 1, 2, 2>(env, p, count, t, extra)
                  : launch_typed_wide<XT, false, 1, 2, 2>(env, p, count, t, extra);
    return f16s ? launch_typed_wide<XT, true, 1, 1, 4>(env, p, count, t, extra)
                : launch_typed_wide<XT, false, 1, 1, 4>(env, p, count, t, extra);
  }
  if (pair)
    return f16s ? launch_typed_wide<XT, true, 2, 2, 2>(env, p, count, t, extra)
                : launch_typed_wide<XT, false, 2, 2, 2>(env, p, count, t, extra);
  return f16s ? launch_typed_wide<XT, true, 2, 1, 4>(env, p, count, t, extra)
              : launch_typed_wide<XT, false, 2, 1, 4>(env, p, count, t, extra);
}

}  // namespace

// True when launch_qgemv_i4 takes this request to the wide kernel, which applies
// env.norm_weight / env.residual itself (the branch of launch_x, restated).
bool qgemv_i4_fuses_neighbours(int count, const LinearTarget* targets, int x_dtype, uint32_t m) {
  if (count < 1 || count > kMaxMulti || m < 5 || m > 16) return false;
  if (x_dtype != KQ_F32 && x_dtype != KQ_F16 && x_dtype != KQ_BF16) return false;
  for (int i = 0; i < count; ++i) {
    const Weight& w = *targets[i].w;
    if (w.layout != kLayoutTiledI4 || w.k != targets[0].w->k || w.scale_dtype != targets[0].w->scale_dtype || w.n == 0) return false;
  }
  return true;
}

bool qgemv_i4_supports(const Weight& w, uint32_t m) {
  return w.layout == kLayoutTiledI4 && m >= 1 && m <= 16;
}

cudaError_t launch_qgemv_i4(const LaunchEnv& env, int count, const LinearTarget* targets,
                            const void* x, int x_dtype, uint32_t m, int* launches) {
  if (count < 1 || count > kMaxMulti || m < 1 || m > 16) return cudaErrorInvalidValue;
  GemvParams p = {};
  p.count = static_cast<uint32_t>(count);
  const uint32_t k = targets[0].w->k;
  const int scale_dtype = targets[0].w->scale_dtype;
  for (int i = 0; i < count; ++i) {
    const Weight& w = *targets[i].w;
    if (w.layout != kLayoutTiledI4 || w.k != k || w.scale_dtype != scale_dtype) return cudaErrorInvalidValue;
    p.w[i] = static_cast<const uint8_t*>(w.data);
    p.bias[i] = targets[i].bias;
    p.out[i] = targets[i].out;
    p.n[i] = w.n;
  }
  p.x = x;
  p.m = m;
  p.k = k;
  const bool f16s = scale_dtype == KQ_F16;
  cudaError_t e;
  switch (x_dtype) {
    case KQ_F32: e = launch_x<float>(env, p, count, targets, f16s, launches); break;
    case KQ_F16: e = launch_x<__half>(env, p, count, targets, f16s, launches); break;
    case KQ_BF16: e = launch_x<__nv_bfloat16>(env, p, count, targets, f16s, launches); break;
    default: return cudaErrorInvalidValue;
  }
  if (e == cudaSuccess && launches) *launches += 1;
  return e;
}

}  // namespace kq
