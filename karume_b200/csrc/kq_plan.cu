// kq_plan — a recorded sequence of quantized linears executed by ONE persistent kernel.
//
// Replaces the reference's baked-plan replay (executeBakedPlan,
// packages/runtime/src/runtime/recipe.ts:462) for plans made of int4 / group-32 linears with
// at most 16 activation rows — a decode step.  Launching those ~130 small, dependent
// matmuls one by one costs more in launch and drain latency than in memory time; here one
// CTA per SM stays resident for the whole plan and the weight stream never stops:
//
//   * every warp owns a static list of work items across ALL ops of the plan (an item = a
//     16-row block x one k-slab of the tiled layout) and streams them in pieces of up to
//     4.6 KB through its private shared-memory ring with cp.async.bulk + mbarrier.  The
//     copies for the next op are issued before the warp waits for the previous op to
//     finish, so HBM keeps streaming through the dependency barriers;
//   * the math per 64-k chunk is the same as in qgemv_i4_kernel (kq_gemv_core.cuh): nibble
//     pairs as binary16 subnormals into mma.sync, hi/lo activation columns, f32 group scale;
//   * an op with few output rows splits K over the warps of ONE CTA (S slabs x 16/S row
//     blocks per CTA round); the S partial sums meet in shared memory and are added in slab
//     order (deterministic, no atomics, no global scratch).  Ops with many rows give every
//     warp a whole row block and store straight from registers;
//   * ops are separated by a grid-wide barrier (all CTAs are co-resident: cooperative
//     launch).  Every wait in this file is bounded: if one gives up, the kernel records a
//     status word, keeps going without blocking, and the host reports KQ_ERR_TIMEOUT.
#include <algorithm>
#include <climits>
#include <type_traits>
#include <utility>
#include <vector>

#include "kq_gemv_core.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kPlanWarps = 16;
constexpr int kSlots = 2;  // ring slots per warp
constexpr uint32_t kOpWindow = 16;  // op descriptors the paired kernel keeps in shared memory
constexpr uint32_t kSpinLimit = 1u << 22;

// What an op does besides out = x . W^T + bias (kq_linear_fused): all of it runs inside the
// paired kernel, in the activation staging (norm) and in the epilogue (the rest).
constexpr uint32_t kOpSwiglu = 1u;  // weights (gate, up): out[0] = silu(x.Wg^T + bg) * (x.Wu^T + bu)
constexpr uint32_t kOpReduce = 2u;  // row-parallel shard: the outputs are added across ranks

struct PlanOpDev {
  const uint8_t* w[kMaxMulti];
  const float* bias[kMaxMulti];
  float* out[kMaxMulti];
  const float* residual[kMaxMulti];  // null, or [m, n] added to the output (may alias it)
  uint32_t n[kMaxMulti];
  uint32_t rb_begin[kMaxMulti + 1];  // prefix sums of n / 16
  uint32_t count;
  uint32_t flags;
  const void* x;
  const float* norm_weight;  // null, or [k]: x is rms-normalised with this weight while it is staged
  float norm_eps;
  uint32_t reduce_index;     // ordinal of this op among the plan's kOpReduce ops
  long long gate_up_delta;   // kOpSwiglu: bytes from the gate weight to the up weight (any distance)
  uint32_t k;
  uint32_t chunks_per_row;   // k / 64
  uint32_t slabs;            // S: k-slabs a row block is split into across the warps of a CTA
  uint32_t slabs_log2;
  uint32_t chunks_per_slab;  // ceil(chunks_per_row / S)
  uint32_t row_blocks;       // 16-row blocks of the op
  uint32_t cta_items;        // ceil(row_blocks / (kPlanWarps / S)): CTA-sized units of work
  uint32_t rounds;           // ceil(cta_items / grid)
  uint32_t rot;              // CTA b works on unit round*grid + (b + rot) % grid
};

struct PlanParams {
  const PlanOpDev* ops;
  uint32_t op_count;
  uint32_t m;
  uint32_t xs_bytes;       // shared memory reserved for the staged activations of one op
  unsigned int* grid_bar;  // arrivals at the inter-op barrier (zeroed before every launch)
  int* status;             // non-zero: a bounded wait gave up
  const FusedCommDev* fcomm;  // exchange areas of the ranks (plans with kOpReduce ops)
  uint32_t reduce_ops;        // how many kOpReduce ops the plan holds
  unsigned long long* trace;  // null, or [cta][op][kTraceSlots] %globaltimer stamps (kq_plan_profile)
};

// Phase stamps one CTA (its thread 0) leaves per op when a plan is profiled.
constexpr uint32_t kTraceSlots = 8;
enum : uint32_t {
  kTraceOpBegin = 0,    // the CTA is done with the previous op
  kTraceBarrier = 1,    // the grid barrier has let it through
  kTraceStaged = 2,     // the activations are staged
  kTraceFirstPiece = 3, // warp 0's first weight piece of the op has landed
  kTraceConsumed = 4,   // warp 0 has consumed the weights of its first round
  kTraceOpEnd = 5       // outputs of the last round stored
};
__device__ __forceinline__ void trace_stamp(const PlanParams& p, uint32_t op, uint32_t slot) {
  if (p.trace != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.trace[(static_cast<size_t>(blockIdx.x) * p.op_count + op) * kTraceSlots + slot] = t;
  }
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One exchange entry = {value, epoch} in ONE aligned 64-bit word, written and polled with scalar
// 64-bit accesses (single-copy atomic: a reader that sees the new epoch sees the value stored
// with it).  Relaxed, system scope: the entry is its own flag.
__device__ __forceinline__ void st_exchange_entry(uint2* p, float value, unsigned int epoch) {
  const unsigned long long word = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(value);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(word) : "memory");
}
__device__ __forceinline__ uint2 ld_exchange_entry(const uint2* p) {
  unsigned long long word;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(p) : "memory");
  return make_uint2(static_cast<uint32_t>(word), static_cast<uint32_t>(word >> 32));
}

// One warp's share of one CTA round of an op.
struct WarpItem {
  const uint8_t* src;  // first chunk of the slab in the tiled layout
  uint32_t nck;        // chunks in the slab (0: nothing to do)
  uint32_t c0;         // first chunk index inside the row (for the staged activations)
  uint32_t rb;         // row block inside the op
  uint32_t wi;         // which weight of the op
  bool row_block_valid;
};

template <uint32_t kCB>
__device__ __forceinline__ WarpItem item_of(const PlanOpDev& o, uint32_t round, uint32_t warp, uint32_t grid,
                                            uint32_t cta) {
  WarpItem it;
  it.nck = 0;
  it.row_block_valid = false;
  it.src = nullptr;
  it.c0 = 0;
  it.rb = 0;
  it.wi = 0;
  uint32_t cta_eff = cta + o.rot;
  if (cta_eff >= grid) cta_eff -= grid;
  const uint32_t unit = round * grid + cta_eff;
  if (unit >= o.cta_items) return it;
  const uint32_t per_cta = kPlanWarps / o.slabs;  // row blocks per CTA round
  const uint32_t sub = warp / o.slabs, slab = warp - sub * o.slabs;
  it.rb = unit * per_cta + sub;
  if (it.rb >= o.row_blocks) return it;
  it.row_block_valid = true;
#pragma unroll
  for (int i = 1; i < kMaxMulti; ++i)
    if (i < static_cast<int>(o.count) && it.rb >= o.rb_begin[i]) it.wi = i;
  it.c0 = slab * o.chunks_per_slab;
  if (it.c0 >= o.chunks_per_row) return it;
  it.nck = min(o.chunks_per_slab, o.chunks_per_row - it.c0);
  it.src = o.w[it.wi] + (static_cast<size_t>(it.rb - o.rb_begin[it.wi]) * o.chunks_per_row + it.c0) * kCB;
  return it;
}

template <typename XT, bool kScaleF16, int kCols, int kSlotChunks, int kG>
__global__ void __launch_bounds__(kPlanWarps * 32, 1)
plan_kernel(const PlanParams p) {
  // kG > 1: kG consecutive scale groups share one 8-column MMA tile (see
  // qgemv_i4_gp_kernel); kG == 1: one group per tile, kCols / 8 tiles.
  static_assert(kG == 1 || kCols == 8, "group packing uses a single tile");
  constexpr int kCpg = 8 / kG;   // MMA columns per group when packing
  constexpr int kCU = kG > 1 ? kG / 2 : 1;  // chunks per unit
  static_assert(kSlotChunks % kCU == 0, "ring pieces hold whole units");
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;  // chunk bytes
  constexpr uint32_t kSlotBytes = kSlotChunks * kCB;
  constexpr int kTiles = kCols / 8;
  constexpr int kAccPerTile = kHasLo ? 2 : 4;
  constexpr int kCorrPerTile = kHasLo ? 1 : 2;
  constexpr int kCorrStride = kG > 1 ? (kHasLo ? kCpg / 2 : kCpg) : (kHasLo ? kCols / 2 : kCols);
  constexpr uint32_t kMask0 = 0x000F000Fu, kMask1 = 0x00F000F0u;

  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t grid = gridDim.x, cta = blockIdx.x;

  // shared memory: [warp rings][mbarriers][staged x][corr][reduction buffers x2]
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t ring = smem_base + warp * (kSlots * kSlotBytes);
  const uint32_t bars = smem_base + kPlanWarps * kSlots * kSlotBytes + warp * (kSlots * 8);
  uint8_t* xs = smem + kPlanWarps * kSlots * kSlotBytes + kPlanWarps * kSlots * 8;
  const uint32_t active_cols = kHasLo ? 2 * p.m : p.m;
  const uint32_t xs_stride = kG > 1 ? kCpg * 64u : active_cols * 64;
  const uint32_t groups_max = p.xs_bytes / xs_stride;
  float* corr = reinterpret_cast<float*>(xs + p.xs_bytes);  // {-8 sum x, 2^-e} pairs, see stage_x
  float* red = corr + groups_max * kCorrStride * 2;  // [2][kPlanWarps][m][16]

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kSlots; ++s) mbar_init(bars + s * 8, 1);
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  // Producer side: start the copy of the next piece (<= kSlotChunks chunks) of this warp's
  // work list, whatever op it belongs to, into the slot sequence number prod_q maps to.
  uint32_t prod_op = 0, prod_round = 0, prod_piece = 0, prod_q = 0;
  auto produce = [&]() {
    while (prod_op < p.op_count) {
      const PlanOpDev& o = p.ops[prod_op];
      if (prod_round >= o.rounds) {
        prod_op += 1;
        prod_round = 0;
        prod_piece = 0;
        continue;
      }
      const WarpItem it = item_of<kCB>(o, prod_round, warp, grid, cta);
      if (it.nck == 0) {
        prod_round += 1;
        prod_piece = 0;
        continue;
      }
      const uint32_t first = prod_piece * kSlotChunks;
      const uint32_t nc = min(static_cast<uint32_t>(kSlotChunks), it.nck - first);
      const uint32_t slot = prod_q & 1u;
      if (lane == 0) {
        mbar_expect_tx(bars + slot * 8, nc * kCB);
        bulk_copy_g2s(ring + slot * kSlotBytes, it.src + static_cast<size_t>(first) * kCB, nc * kCB, bars + slot * 8);
      }
      prod_q += 1;
      prod_piece += 1;
      if (prod_piece * kSlotChunks >= it.nck) {
        prod_piece = 0;
        prod_round += 1;
      }
      return;
    }
  };
#pragma unroll
  for (int s = 0; s < kSlots; ++s) produce();

  // Persistent per-lane state of the MMA operands (see qgemv_i4_kernel).
  uint4 bfrag[kTiles];
  float cterm[kTiles][kCorrPerTile], cinv[kTiles][kCorrPerTile];
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

  // Group packing: the group (inside a unit) and activation row(s) of this lane's two C
  // columns, the group whose activations it feeds the MMAs with, one register set per group.
  const uint32_t jl = kG > 1 ? (2u * t) / kCpg : 0u;
  const uint32_t tl = kG > 1 ? t % (kCpg / 2) : t;
  uint4 bset[kG];
  bool load_bset[kG];
  float gterm[kCorrPerTile], ginv[kCorrPerTile];
  bool load_g[kCorrPerTile];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    bset[j] = make_uint4(0, 0, 0, 0);
    load_bset[j] = kG > 1 && (g % kCpg) < active_cols && g / kCpg == static_cast<uint32_t>(j);
  }
#pragma unroll
  for (int j = 0; j < kCorrPerTile; ++j) {
    gterm[j] = 0.0f;
    ginv[j] = 0.0f;
    load_g[j] = (kHasLo ? tl : 2 * tl + j) < p.m;
  }
  const uint32_t gcorr_lane = static_cast<uint32_t>(__cvta_generic_to_shared(corr)) +
                              (jl * kCorrStride + (kHasLo ? tl : 2 * tl)) * 8;
  const uint32_t gscale_off = (jl >> 1) * kCB + kChunkWeightBytes + g * (4 * kScaleBytes) + (jl & 1u) * (2 * kScaleBytes);

  uint32_t cons_q = 0, red_buf = 0;
  for (uint32_t op = 0; op < p.op_count; ++op) {
    const PlanOpDev& o = p.ops[op];
    if (op > 0) {
      // every output of the previous op must be complete and visible before x is read
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(p.grid_bar, 1u);
        const unsigned int target = op * grid;
        uint32_t spins = 0;
        while (ld_acquire_gpu(p.grid_bar) < target) {
          if (++spins > kSpinLimit) {
            *reinterpret_cast<volatile int*>(p.status) = 1;
            break;
          }
        }
        __threadfence();
      }
      __syncthreads();
    }
    // stage the op's whole activation block (it fits: checked when the plan was built)
    stage_x<XT, kHasLo, kCorrStride, true>(static_cast<const XT*>(o.x), p.m, o.k, 0, o.k >> 5, xs, xs_stride, corr);
    __syncthreads();

    const uint32_t slabs = o.slabs;
    for (uint32_t round = 0; round < o.rounds; ++round) {
      const WarpItem it = item_of<kCB>(o, round, warp, grid, cta);
      float acc[kTiles][kAccPerTile];
#pragma unroll
      for (int i = 0; i < kTiles; ++i)
#pragma unroll
        for (int j = 0; j < kAccPerTile; ++j) acc[i][j] = 0.0f;

      for (uint32_t first = 0; first < it.nck; first += kSlotChunks) {
        const uint32_t nc = min(static_cast<uint32_t>(kSlotChunks), it.nck - first);
        const uint32_t slot = cons_q & 1u, parity = (cons_q >> 1) & 1u;
        {
          uint32_t spins = 0;
          while (!mbar_try_wait(bars + slot * 8, parity)) {
            if (++spins > kSpinLimit) {
              *reinterpret_cast<volatile int*>(p.status) = 2;
              break;
            }
          }
        }
        const uint32_t slot_addr = ring + slot * kSlotBytes;
        const uint32_t group0 = 2 * (it.c0 + first);
        if constexpr (kG > 1) {
          const uint32_t unit0 = (it.c0 + first) / kCU;
#pragma unroll 2
          for (uint32_t c = 0; c < nc; c += kCU) {
            const uint32_t chunk_addr = slot_addr + c * kCB;
            const uint32_t unit = unit0 + c / kCU;
            uint4 wq[kCU];
#pragma unroll
            for (int cc = 0; cc < kCU; ++cc)
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(wq[cc].x), "=r"(wq[cc].y), "=r"(wq[cc].z), "=r"(wq[cc].w)
                           : "r"(chunk_addr + cc * kCB + lane * 16));
            float2 s;  // rows g, g + 8 of the lane's own group
            if constexpr (kScaleF16) {
              uint32_t raw;
              asm volatile("ld.shared.u32 %0, [%1];" : "=r"(raw) : "r"(chunk_addr + gscale_off));
              s = __half22float2(*reinterpret_cast<const __half2*>(&raw));
            } else {
              asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(s.x), "=f"(s.y) : "r"(chunk_addr + gscale_off));
            }
#pragma unroll
            for (int j = 0; j < kG; ++j) lds_v4_if(bset[j], xs_lane + unit * 512, load_bset[j]);
#pragma unroll
            for (int j = 0; j < kCorrPerTile; ++j)
              lds_v2f_if(gterm[j], ginv[j], gcorr_lane + (unit * (kG * kCorrStride) + j) * 8, load_g[j]);
            float cf[4];
#pragma unroll
            for (int j = 0; j < kG; ++j) {
              const uint32_t wa = (j & 1) ? wq[j >> 1].z : wq[j >> 1].x;  // row g
              const uint32_t wb = (j & 1) ? wq[j >> 1].w : wq[j >> 1].y;  // row g + 8
              const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
              const uint32_t a0[4] = {wa & kMask0, wb & kMask0, wa & kMask1, wb & kMask1};
              const uint32_t a1[4] = {wa8 & kMask0, wb8 & kMask0, wa8 & kMask1, wb8 & kMask1};
              if (j == 0) mma_f16_zero(cf, a0, bset[j].x, bset[j].y);
              else mma_f16(cf, a0, bset[j].x, bset[j].y);
              mma_f16(cf, a1, bset[j].z, bset[j].w);
            }
            if constexpr (kHasLo) {
              acc[0][0] = fmaf(s.x, fmaf(cf[0] + cf[1], ginv[0], gterm[0]), acc[0][0]);
              acc[0][1] = fmaf(s.y, fmaf(cf[2] + cf[3], ginv[0], gterm[0]), acc[0][1]);
            } else {
              acc[0][0] = fmaf(s.x, fmaf(cf[0], ginv[0], gterm[0]), acc[0][0]);
              acc[0][1] = fmaf(s.x, fmaf(cf[1], ginv[1], gterm[1]), acc[0][1]);
              acc[0][2] = fmaf(s.y, fmaf(cf[2], ginv[0], gterm[0]), acc[0][2]);
              acc[0][3] = fmaf(s.y, fmaf(cf[3], ginv[1], gterm[1]), acc[0][3]);
            }
          }
        } else {
#pragma unroll 2
        for (uint32_t c = 0; c < nc; ++c) {
          const uint32_t chunk_addr = slot_addr + c * kCB;
          uint4 wq;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(wq.x), "=r"(wq.y), "=r"(wq.z), "=r"(wq.w) : "r"(chunk_addr + lane * 16));
          float2 sc[2];  // [group]: .x = row g, .y = row g + 8
          if constexpr (kScaleF16) {
            uint2 raw;
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(raw.x), "=r"(raw.y)
                         : "r"(chunk_addr + kChunkWeightBytes + g * 8));
            sc[0] = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            sc[1] = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
          } else {
            uint4 raw;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                         : "r"(chunk_addr + kChunkWeightBytes + g * 16));
            sc[0] = make_float2(__uint_as_float(raw.x), __uint_as_float(raw.y));
            sc[1] = make_float2(__uint_as_float(raw.z), __uint_as_float(raw.w));
          }
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const uint32_t lg = group0 + 2 * c + jj;
#pragma unroll
            for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
              lds_v4_if(bfrag[tile_m], xs_lane + lg * xs_stride + tile_m * 512, load_b[tile_m]);
#pragma unroll
              for (int j = 0; j < kCorrPerTile; ++j)
                lds_v2f_if(cterm[tile_m][j], cinv[tile_m][j],
                           corr_lane + (lg * kCorrStride + tile_m * (kHasLo ? 4 : 8) + j) * 8, load_c[tile_m][j]);
            }
            const uint32_t wa = jj ? wq.z : wq.x;  // row g
            const uint32_t wb = jj ? wq.w : wq.y;  // row g + 8
            const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
            const uint32_t a0[4] = {wa & kMask0, wb & kMask0, wa & kMask1, wb & kMask1};
            const uint32_t a1[4] = {wa8 & kMask0, wb8 & kMask0, wa8 & kMask1, wb8 & kMask1};
            const float2 s = sc[jj];
#pragma unroll
            for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
              float cf[4];
              mma_f16_zero(cf, a0, bfrag[tile_m].x, bfrag[tile_m].y);
              mma_f16(cf, a1, bfrag[tile_m].z, bfrag[tile_m].w);
              if constexpr (kHasLo) {
                acc[tile_m][0] = fmaf(s.x, fmaf(cf[0] + cf[1], cinv[tile_m][0], cterm[tile_m][0]), acc[tile_m][0]);
                acc[tile_m][1] = fmaf(s.y, fmaf(cf[2] + cf[3], cinv[tile_m][0], cterm[tile_m][0]), acc[tile_m][1]);
              } else {
                acc[tile_m][0] = fmaf(s.x, fmaf(cf[0], cinv[tile_m][0], cterm[tile_m][0]), acc[tile_m][0]);
                acc[tile_m][1] = fmaf(s.x, fmaf(cf[1], cinv[tile_m][1], cterm[tile_m][1]), acc[tile_m][1]);
                acc[tile_m][2] = fmaf(s.y, fmaf(cf[2], cinv[tile_m][0], cterm[tile_m][0]), acc[tile_m][2]);
                acc[tile_m][3] = fmaf(s.y, fmaf(cf[3], cinv[tile_m][1], cterm[tile_m][1]), acc[tile_m][3]);
              }
            }
          }
        }
        }
        __syncwarp();  // every lane has read the slot: it can take the next piece
        produce();
        cons_q += 1;
      }

      // ---- this round's outputs ------------------------------------------------------
      if constexpr (kG > 1) {
        // lanes whose C columns belong to different groups hold partial sums of the same outputs
#pragma unroll
        for (int j = 0; j < kAccPerTile; ++j) {
          if constexpr (kG == 4) acc[0][j] += __shfl_xor_sync(0xffffffffu, acc[0][j], 1);
          acc[0][j] += __shfl_xor_sync(0xffffffffu, acc[0][j], 2);
        }
      }
      const bool owner = jl == 0;  // always true without group packing
      const uint32_t local_row = (it.rb - o.rb_begin[it.wi]) * 16u;  // first row of the block inside its weight
      const uint32_t n_i = o.n[it.wi];
      float* out = o.out[it.wi];
      const float* bias = o.bias[it.wi];
      if (slabs == 1) {
        if (it.nck != 0 && owner) {
#pragma unroll
          for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
#pragma unroll
            for (int j = 0; j < (kHasLo ? 1 : 2); ++j) {
              const uint32_t mm = kHasLo ? tile_m * 4 + tl : tile_m * 8 + 2 * tl + j;
              if (mm >= p.m) continue;
              const float va = acc[tile_m][kHasLo ? 0 : j];
              const float vb = acc[tile_m][kHasLo ? 1 : 2 + j];
              out[static_cast<size_t>(mm) * n_i + local_row + g] = fmaf(va, kUnscale, bias[local_row + g]);
              out[static_cast<size_t>(mm) * n_i + local_row + g + 8] = fmaf(vb, kUnscale, bias[local_row + g + 8]);
            }
          }
        }
        continue;
      }
      // K was split over `slabs` warps of this CTA: meet in shared memory, add in slab order.
      float* mine = red + (static_cast<size_t>(red_buf) * kPlanWarps + warp) * p.m * 16;
#pragma unroll
      for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
#pragma unroll
        for (int j = 0; j < (kHasLo ? 1 : 2); ++j) {
          const uint32_t mm = kHasLo ? tile_m * 4 + tl : tile_m * 8 + 2 * tl + j;
          if (mm >= p.m || !owner) continue;
          mine[mm * 16 + g] = acc[tile_m][kHasLo ? 0 : j];          // zeros when the warp had no chunks
          mine[mm * 16 + g + 8] = acc[tile_m][kHasLo ? 1 : 2 + j];
        }
      }
      __syncthreads();
      const uint32_t sub = warp / slabs;
      if (warp - sub * slabs == 0 && it.row_block_valid) {
        const float* first_slab = red + (static_cast<size_t>(red_buf) * kPlanWarps + warp) * p.m * 16;
        for (uint32_t idx = lane; idx < 16u * p.m; idx += 32) {
          float total = 0.0f;
          for (uint32_t s = 0; s < slabs; ++s) total += first_slab[static_cast<size_t>(s) * p.m * 16 + idx];
          const uint32_t mm = idx >> 4, r = idx & 15u;
          out[static_cast<size_t>(mm) * n_i + local_row + r] = fmaf(total, kUnscale, bias[local_row + r]);
        }
      }
      red_buf ^= 1u;  // the next round writes the other buffer; this one is re-used two rounds on
    }
  }
}

// ---- paired kernel: two row blocks per warp, group-packed MMA tiles ---------------------
// The fast path for one or two activation rows (at most 4 MMA columns).  Differences from
// plan_kernel above:
//   * a warp's work item is a PAIR of adjacent 16-row blocks over one k-slab; both blocks use
//     the same staged activations, so one set of shared loads (and their predicates and
//     addresses) feeds two independent MMA chains;
//   * kG scale groups share one C tile (see qgemv_i4_gp_kernel), so a lane scales only the
//     group its two C columns belong to;
//   * a ring slot holds the same kPiece chunks of k for both blocks ([block 0][block 1]);
//     full pieces are consumed by straight-line code with immediate address offsets;
//   * the producer keeps its position inside the current item in registers and touches the
//     op descriptor only when it moves to the next item.
template <int... kIs, typename F>
__device__ __forceinline__ void static_for_impl(std::integer_sequence<int, kIs...>, F&& f) {
  (f(std::integral_constant<int, kIs>{}), ...);
}
template <int kN, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  static_for_impl(std::make_integer_sequence<int, kN>{}, static_cast<F&&>(f));
}

template <int kOff>
__device__ __forceinline__ uint4 lds_v4_at(uint32_t base) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(base), "n"(kOff));
  return v;
}
template <int kOff>
__device__ __forceinline__ uint32_t lds_u32_at(uint32_t base) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(base), "n"(kOff));
  return v;
}
template <int kOff>
__device__ __forceinline__ uint2 lds_v2_at(uint32_t base) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(base), "n"(kOff));
  return v;
}
template <int kOff>
__device__ __forceinline__ void lds_v4_if_at(uint4& v, uint32_t base, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%6];\n\t}"
               : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
               : "r"(base), "r"(static_cast<uint32_t>(pred)), "n"(kOff));
}
template <int kOff>
__device__ __forceinline__ void lds_v2f_if_at(float& a, float& b, uint32_t base, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\t@p ld.shared.v2.f32 {%0,%1}, [%2+%4];\n\t}"
               : "+f"(a), "+f"(b) : "r"(base), "r"(static_cast<uint32_t>(pred)), "n"(kOff));
}

// Sum over the k-slabs of one output, slab order fixed: ((s0 + s1) + (s2 + s3)) + ... per group of
// four, groups in ascending order (slabs is a power of two >= 2).  Four independent loads per
// step instead of a chain of dependent load-add pairs.
__device__ __forceinline__ float sum_slabs(const float* first, uint32_t slabs, uint32_t stride) {
  if (slabs == 2) return first[0] + first[stride];
  float total = 0.0f;
  for (uint32_t sl = 0; sl < slabs; sl += 4) {
    const float a = first[static_cast<size_t>(sl) * stride], b = first[static_cast<size_t>(sl + 1) * stride];
    const float c = first[static_cast<size_t>(sl + 2) * stride], d = first[static_cast<size_t>(sl + 3) * stride];
    total += (a + b) + (c + d);
  }
  return total;
}

// ---- finishing the outputs of ops with fused neighbours ---------------------------------
// out = partial sum (scaled back) [summed over the ranks] + bias [+ residual], each addition
// rounded to f32 like the reference's node sequence linear -> add; or silu(gate) * up.
//
// Cross-rank sum (kOpReduce): every lane PUSHES its finished partial sums into the exchange
// area of every peer as {value, epoch} entries (slot = epoch parity, source = this rank), then
// polls (bounded) its own area until the peers' entries carry this epoch and adds the ranks'
// values in rank order, so all ranks hold the same bits.  The k-th reduce op of a launch uses
// epoch base + 1 + k, where base is what the previous launch (of a plan or of kq_linear_reduce)
// left in the exchange area; the last CTA of a launch advances it.  Entries of consecutive
// epochs alternate between two slots, and the grid barrier between ops keeps every rank within
// one exchange of its peers, so an unread entry is never overwritten.
constexpr int kFinish = 4;  // outputs finished per call
__device__ __forceinline__ void exchange_sum(const FusedCommDev* fcp, int* status, unsigned int epoch,
                                             float (&val)[kFinish], const uint32_t (&off)[kFinish], uint32_t vmask) {
  const FusedCommDev& fc = *fcp;
  const uint32_t me = fc.rank, world = fc.world;
  const uint64_t slot_entries = kFusedSlotBytes / 8;
  const uint64_t parity_base = static_cast<uint64_t>(epoch & 1u) * kFusedMaxWorld;
  for (uint32_t r = 0; r < world; ++r) {
    if (r == me) continue;
    uint2* dst = reinterpret_cast<uint2*>(fc.base[r] + fc.data_off) + (parity_base + me) * slot_entries;
#pragma unroll
    for (int i = 0; i < kFinish; ++i)
      if (vmask & (1u << i)) st_exchange_entry(dst + off[i], val[i], epoch);
  }
#pragma unroll
  for (int i = 0; i < kFinish; ++i) {
    if (!(vmask & (1u << i))) continue;
    float sum = 0.0f;
    for (uint32_t r = 0; r < world; ++r) {
      if (r == me) {
        sum += val[i];
        continue;
      }
      const uint2* src = reinterpret_cast<const uint2*>(fc.base[me] + fc.data_off) + (parity_base + r) * slot_entries + off[i];
      uint2 e;
      uint32_t spins = 0;
      while (true) {
        e = ld_exchange_entry(src);
        if (e.y == epoch) break;
        if (++spins > kSpinLimit) {
          *reinterpret_cast<volatile int*>(status) = 3;
          break;
        }
      }
      sum += __uint_as_float(e.x);
    }
    val[i] = sum;
  }
}

__device__ __forceinline__ void finish_values(const PlanOpDev* o, uint32_t wi, float (&val)[kFinish],
                                              const uint32_t (&off)[kFinish], const float (&bsv)[kFinish], uint32_t vmask,
                                              const FusedCommDev* fc, int* status, bool have_residual0 = false,
                                              float residual0 = 0.0f) {
  if (vmask == 0) return;
#pragma unroll
  for (int i = 0; i < kFinish; ++i) val[i] *= kUnscale;
  if (o->flags & kOpReduce) {
    // the epoch word keeps the launch's base until the last CTA of the launch has finished
    const unsigned int epoch_base = *reinterpret_cast<volatile unsigned int*>(fc->epoch);
    exchange_sum(fc, status, epoch_base + 1u + o->reduce_index, val, off, vmask);
  }
  const float* residual = o->residual[wi];
  float* out = o->out[wi];
#pragma unroll
  for (int i = 0; i < kFinish; ++i) {
    if (!(vmask & (1u << i))) continue;
    float v = __fadd_rn(val[i], bsv[i]);
    if (residual != nullptr) v = __fadd_rn(v, (i == 0 && have_residual0) ? residual0 : residual[off[i]]);
    out[off[i]] = v;
  }
}

// One lane's outputs of an unsplit pair: rows `row`, row + 8 of the first block (a0, a1) and of
// the second block (b0, b1) for activation row mm.  For the SiLU gate the first block is the
// gate and the second the up projection of the same 16 output rows.
__device__ __noinline__ void finish_fused_lane(const PlanOpDev* o, uint32_t wi, uint32_t mm, uint32_t row, float a0, float a1,
                                               float b0, float b1, float bias0, float bias1, float bias2, float bias3,
                                               const FusedCommDev* fc, int* status) {
  const uint32_t n_i = o->n[wi];
  if (o->flags & kOpSwiglu) {
    float* dst = o->out[0] + static_cast<size_t>(mm) * n_i + row;
    dst[0] = silu_mul(fmaf(a0, kUnscale, bias0), fmaf(b0, kUnscale, bias2));
    dst[8] = silu_mul(fmaf(a1, kUnscale, bias1), fmaf(b1, kUnscale, bias3));
    return;
  }
  const uint32_t base = mm * n_i + row;
  float val[kFinish] = {a0, a1, b0, b1};
  const uint32_t off[kFinish] = {base, base + 8, base + 16, base + 24};
  const float bsv[kFinish] = {bias0, bias1, bias2, bias3};
  finish_values(o, wi, val, off, bsv, 0xFu, fc, status);
}

// The reducing warp of a pair whose K range was split over `slabs` warps: adds the slabs' partial
// sums ([slab][block][m][16] in shared memory) in slab order and finishes the 32 (SiLU gate: 16)
// output rows x m.
__device__ __noinline__ void finish_fused_slabs(const PlanOpDev* o, uint32_t wi, const float* first_slab, uint32_t slabs,
                                                uint32_t m, uint32_t local_row, uint32_t lane, float bias_lane,
                                                float residual_lane, const FusedCommDev* fc, int* status) {
  const uint32_t n_i = o->n[wi], slab_stride = 2 * m * 16;
  if (o->flags & kOpSwiglu) {
    const float* bias_g = o->bias[0];
    const float* bias_u = o->bias[1];
    for (uint32_t idx = lane; idx < 16u * m; idx += 32) {
      const uint32_t mm = idx >> 4, rr = idx & 15u;
      const float tg = sum_slabs(first_slab + mm * 16 + rr, slabs, slab_stride);
      const float tu = sum_slabs(first_slab + (m + mm) * 16 + rr, slabs, slab_stride);
      const uint32_t row = local_row + rr;
      o->out[0][static_cast<size_t>(mm) * n_i + row] = silu_mul(fmaf(tg, kUnscale, bias_g[row]), fmaf(tu, kUnscale, bias_u[row]));
    }
    return;
  }
  const float* bias = o->bias[wi];
  for (uint32_t first = 0; first < 32u * m; first += 32u * kFinish) {
    float val[kFinish], bsv[kFinish];
    uint32_t off[kFinish];
    uint32_t vmask = 0;
#pragma unroll
    for (int i = 0; i < kFinish; ++i) {
      const uint32_t idx = first + lane + 32u * i;
      val[i] = 0.0f;
      bsv[i] = 0.0f;
      off[i] = 0u;
      if (idx < 32u * m) {
        const float total = sum_slabs(first_slab + idx, slabs, slab_stride);
        const uint32_t r = idx / (m * 16), rem = idx - r * (m * 16);
        const uint32_t mm = rem >> 4, row = local_row + r * 16 + (rem & 15u);
        val[i] = total;
        off[i] = mm * n_i + row;
        bsv[i] = (m == 1 && idx == lane) ? bias_lane : bias[row];  // fetched before the weights were consumed
        vmask |= 1u << i;
      }
    }
    finish_values(o, wi, val, off, bsv, vmask, fc, status, m == 1 && first == 0, residual_lane);
  }
}

constexpr int32_t kStrideInDescriptor = INT32_MIN;  // PairItem::row_stride16: see PlanOpDev::gate_up_delta

struct PairItem {
  const uint8_t* src;  // first chunk of the slab of the pair's first row block
  int32_t row_stride16;  // 16-byte units from a chunk of the first block to the same chunk of the second
  uint32_t nck;        // chunks in the slab (0: nothing to do)
  uint32_t c0;         // first chunk index inside the row
  uint32_t rb;         // first row block of the pair, inside the op
  uint32_t wi;         // which weight of the op
  bool valid;          // the pair exists (its outputs are stored)
};

template <uint32_t kCB>
__device__ __forceinline__ PairItem pair_item_of(const PlanOpDev& o, uint32_t round, uint32_t warp, uint32_t grid,
                                                 uint32_t cta) {
  PairItem it;
  it.src = nullptr;
  it.row_stride16 = 0;
  it.nck = 0;
  it.c0 = 0;
  it.rb = 0;
  it.wi = 0;
  it.valid = false;
  uint32_t cta_eff = cta + o.rot;
  if (cta_eff >= grid) cta_eff -= grid;
  const uint32_t unit = round * grid + cta_eff;
  if (unit >= o.cta_items) return it;
  const uint32_t sub = warp >> o.slabs_log2, slab = warp & (o.slabs - 1u);
  const uint32_t pair = unit * (static_cast<uint32_t>(kPlanWarps) >> o.slabs_log2) + sub;
  const bool swiglu = (o.flags & kOpSwiglu) != 0;
  // plain op: two adjacent row blocks of one weight; SiLU gate: block `pair` of the gate weight
  // and the same block of the up weight (row_blocks counts the blocks of ONE of them)
  it.rb = swiglu ? pair : 2u * pair;
  if (it.rb >= o.row_blocks) return it;
  it.valid = true;
  if (!swiglu) {
#pragma unroll
    for (int i = 1; i < kMaxMulti; ++i)
      if (i < static_cast<int>(o.count) && it.rb >= o.rb_begin[i]) it.wi = i;
  }
  it.c0 = slab * o.chunks_per_slab;
  if (it.c0 >= o.chunks_per_row) return it;
  it.nck = min(o.chunks_per_slab, o.chunks_per_row - it.c0);
  // (the gate and the up weight are separate allocations, any distance apart: the producer
  // reads that distance from the descriptor instead of carrying 64 bits of it in a register)
  it.row_stride16 = swiglu ? kStrideInDescriptor : static_cast<int32_t>(o.chunks_per_row * (kCB / 16));
  it.src = o.w[it.wi] + (static_cast<size_t>(it.rb - o.rb_begin[it.wi]) * o.chunks_per_row + it.c0) * kCB;
  return it;
}

template <typename XT, bool kScaleF16, int kG, int kPiece, int kNS>
__global__ void __launch_bounds__(kPlanWarps * 32, 1)
plan_pair_kernel(const PlanParams p) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;
  constexpr int kCpg = 8 / kG;          // MMA columns per group
  constexpr int kCU = kG / 2;           // chunks per unit
  constexpr int kPieceUnits = kPiece / kCU;
  constexpr uint32_t kSlotBytes = 2u * kPiece * kCB;  // both row blocks
  constexpr int kAcc = kHasLo ? 2 : 4;
  constexpr int kCorr = kHasLo ? 1 : 2;
  constexpr int kCorrStride = kHasLo ? kCpg / 2 : kCpg;
  constexpr uint32_t kMask0 = 0x000F000Fu, kMask1 = 0x00F000F0u;
  static_assert(kG == 2 || kG == 4, "units of two or four groups");
  static_assert(kPiece % kCU == 0, "pieces hold whole units");

  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t grid = gridDim.x, cta = blockIdx.x;

  // shared memory: [warp rings][mbarriers][staged x][corr][reduction buffers x2]
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t ring = smem_base + warp * (kNS * kSlotBytes);
  const uint32_t bars = smem_base + kPlanWarps * kNS * kSlotBytes + warp * (kNS * 8);
  uint8_t* xs = smem + kPlanWarps * kNS * kSlotBytes + kPlanWarps * kNS * 8;
  const uint32_t active_cols = kHasLo ? 2 * p.m : p.m;
  constexpr uint32_t kXsStride = kCpg * 64u;
  const uint32_t groups_max = p.xs_bytes / kXsStride;
  float* corr = reinterpret_cast<float*>(xs + p.xs_bytes);  // {-8 sum x, 2^-e} pairs, see stage_x
  float* red = corr + groups_max * kCorrStride * 2;  // [2][kPlanWarps][2][m][16]
  // A window of op descriptors in shared memory (entry i lives in slot i % kOpWindow): the
  // producer and the consumer read them every item, and a chain of dependent global loads
  // there would sit on every warp's critical path.
  PlanOpDev* win = reinterpret_cast<PlanOpDev*>(
      (reinterpret_cast<uintptr_t>(red + 2 * kPlanWarps * 2 * p.m * 16) + 15) & ~static_cast<uintptr_t>(15));
  auto fill_window = [&](uint32_t idx) {
    if (idx >= p.op_count) return;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(p.ops + idx);
    uint32_t* dst = reinterpret_cast<uint32_t*>(win + idx % kOpWindow);
    for (uint32_t i = threadIdx.x; i < sizeof(PlanOpDev) / 4; i += blockDim.x) dst[i] = __ldg(src + i);
  };
  for (uint32_t i = 0; i + 2 <= kOpWindow; ++i) fill_window(i);  // entries 0 .. kOpWindow - 2
  uint32_t cur_op = 0;  // the op this warp is working on; entries up to cur_op + kOpWindow - 2 are valid
  auto desc = [&](uint32_t idx) -> const PlanOpDev& {
    return idx + 2 <= cur_op + kOpWindow ? win[idx % kOpWindow] : p.ops[idx];
  };

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kNS; ++s) mbar_init(bars + s * 8, 1);
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  // ---- producer -------------------------------------------------------------------------
  uint32_t prod_op = 0, prod_round = 0, prod_q = 0, prod_left = 0;
  int32_t prod_stride16 = 0;
  const uint8_t* prod_src = nullptr;
  auto produce = [&]() {
    while (prod_left == 0) {  // move to this warp's next item, whatever op it belongs to
      if (prod_op >= p.op_count) return;
      const PlanOpDev& o = desc(prod_op);
      if (prod_round >= o.rounds) {
        prod_op += 1;
        prod_round = 0;
        continue;
      }
      const PairItem it = pair_item_of<kCB>(o, prod_round, warp, grid, cta);
      prod_round += 1;
      prod_left = it.nck;
      prod_src = it.src;
      prod_stride16 = it.row_stride16;
    }
    const uint32_t nc = min(static_cast<uint32_t>(kPiece), prod_left);
    const uint32_t slot = prod_q & (kNS - 1);
    if (lane == 0) {
      mbar_expect_tx(bars + slot * 8, 2u * nc * kCB);
      bulk_copy_g2s(ring + slot * kSlotBytes, prod_src, nc * kCB, bars + slot * 8);
      const long long delta = prod_stride16 != kStrideInDescriptor ? static_cast<long long>(prod_stride16) * 16
                                                                   : desc(prod_op).gate_up_delta;
      bulk_copy_g2s(ring + slot * kSlotBytes + kPiece * kCB, prod_src + delta, nc * kCB, bars + slot * 8);
    }
    prod_src += nc * kCB;
    prod_left -= nc;
    prod_q += 1;
  };
#pragma unroll
  for (int s = 0; s < kNS; ++s) produce();

  // ---- per-lane constants of the packed MMA tile -----------------------------------------
  const uint32_t jl = (2u * t) / kCpg;      // group (inside a unit) of this lane's two C columns
  const uint32_t tl = t % (kCpg / 2);       // which activation row(s) inside that group
  uint4 bset[kG];
  bool load_bset[kG];
  float gterm[kCorr], ginv[kCorr];
  bool load_g[kCorr];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    bset[j] = make_uint4(0, 0, 0, 0);
    load_bset[j] = (g % kCpg) < active_cols && g / kCpg == static_cast<uint32_t>(j);
  }
#pragma unroll
  for (int j = 0; j < kCorr; ++j) {
    gterm[j] = 0.0f;
    ginv[j] = 0.0f;
    load_g[j] = (kHasLo ? tl : 2 * tl + j) < p.m;
  }
  const uint32_t xs_lane = static_cast<uint32_t>(__cvta_generic_to_shared(xs)) + lane * 16;
  const uint32_t corr_lane = static_cast<uint32_t>(__cvta_generic_to_shared(corr)) +
                             (jl * kCorrStride + (kHasLo ? tl : 2 * tl)) * 8;
  const uint32_t scale_lane = (jl >> 1) * kCB + kChunkWeightBytes + g * (4 * kScaleBytes) + (jl & 1u) * (2 * kScaleBytes);

  float acc[2][kAcc];

  // One unit (kG groups) of both row blocks.  kU selects immediate offsets; callers that
  // cannot unroll pass kU = 0 and pre-advanced base addresses.
  auto unit_step = [&](auto ku, uint32_t w_base, uint32_t s_base, uint32_t xs_base, uint32_t corr_base) {
    constexpr int kU = decltype(ku)::value;
    uint4 wq[2][kCU];
    float2 sc[2];
    static_for<2>([&](auto kr) {
      constexpr int kR = decltype(kr)::value;
      constexpr int kChunk0 = kR * kPiece + kU * kCU;  // first chunk of the unit inside the slot
      wq[kR][0] = lds_v4_at<kChunk0 * kCB>(w_base);
      if constexpr (kCU == 2) wq[kR][1] = lds_v4_at<(kChunk0 + 1) * kCB>(w_base);
      if constexpr (kScaleF16) {
        const uint32_t raw = lds_u32_at<kChunk0 * kCB>(s_base);
        sc[kR] = __half22float2(*reinterpret_cast<const __half2*>(&raw));
      } else {
        const uint2 raw = lds_v2_at<kChunk0 * kCB>(s_base);
        sc[kR] = make_float2(__uint_as_float(raw.x), __uint_as_float(raw.y));
      }
    });
#pragma unroll
    for (int j = 0; j < kG; ++j) lds_v4_if_at<kU * 512>(bset[j], xs_base, load_bset[j]);
    static_for<kCorr>([&](auto kj) {
      constexpr int kJ = decltype(kj)::value;
      lds_v2f_if_at<(kU * kG * kCorrStride + kJ) * 8>(gterm[kJ], ginv[kJ], corr_base, load_g[kJ]);
    });
    float cf[2][4];
#pragma unroll
    for (int j = 0; j < kG; ++j) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint4 wv = wq[r][j >> 1];
        const uint32_t wa = (j & 1) ? wv.z : wv.x;  // row g
        const uint32_t wb = (j & 1) ? wv.w : wv.y;  // row g + 8
        const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
        const uint32_t a0[4] = {wa & kMask0, wb & kMask0, wa & kMask1, wb & kMask1};
        const uint32_t a1[4] = {wa8 & kMask0, wb8 & kMask0, wa8 & kMask1, wb8 & kMask1};
        if (j == 0) mma_f16_zero(cf[r], a0, bset[j].x, bset[j].y);
        else mma_f16(cf[r], a0, bset[j].x, bset[j].y);
        mma_f16(cf[r], a1, bset[j].z, bset[j].w);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if constexpr (kHasLo) {
        acc[r][0] = fmaf(sc[r].x, fmaf(cf[r][0] + cf[r][1], ginv[0], gterm[0]), acc[r][0]);
        acc[r][1] = fmaf(sc[r].y, fmaf(cf[r][2] + cf[r][3], ginv[0], gterm[0]), acc[r][1]);
      } else {
        acc[r][0] = fmaf(sc[r].x, fmaf(cf[r][0], ginv[0], gterm[0]), acc[r][0]);
        acc[r][1] = fmaf(sc[r].x, fmaf(cf[r][1], ginv[1], gterm[1]), acc[r][1]);
        acc[r][2] = fmaf(sc[r].y, fmaf(cf[r][2], ginv[0], gterm[0]), acc[r][2]);
        acc[r][3] = fmaf(sc[r].y, fmaf(cf[r][3], ginv[1], gterm[1]), acc[r][3]);
      }
    }
  };

  uint32_t cons_q = 0, red_buf = 0;
  for (uint32_t op = 0; op < p.op_count; ++op) {
    // Nothing about the first item depends on the previous op: look it up before the wait.
    const PairItem first_item = pair_item_of<kCB>(win[op % kOpWindow], 0, warp, grid, cta);
    trace_stamp(p, op, kTraceOpBegin);
    if (op > 0) {
      // Slot (op - 2) % kOpWindow is dead: every warp passed the barrier of op - 1.
      fill_window(op + kOpWindow - 2);
      // every output of the previous op must be complete and visible before x is read
      __syncthreads();
      if (threadIdx.x == 0) {
        // release: the CTA's stores (ordered before this by the barrier above) become visible
        // to whoever acquires the counter
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.grid_bar) : "memory");
        const unsigned int target = op * grid;
        uint32_t spins = 0;
        while (ld_acquire_gpu(p.grid_bar) < target) {
          if (++spins > kSpinLimit) {
            *reinterpret_cast<volatile int*>(p.status) = 1;
            break;
          }
        }
      }
      __syncthreads();
    }
    cur_op = op;
    const PlanOpDev& o = win[op % kOpWindow];
    trace_stamp(p, op, kTraceBarrier);
    if (o.norm_weight != nullptr) {
      // no reduction of the previous op is in flight any more: its buffers serve as scratch
      float* scratch = red + static_cast<size_t>(red_buf) * kPlanWarps * (2 * p.m * 16);
      stage_x_rms_norm<XT, kHasLo, kCorrStride, true, 4, 4>(static_cast<const XT*>(o.x), o.norm_weight, o.norm_eps, p.m, o.k,
                                                            xs, kXsStride, corr, scratch, scratch + kPlanWarps * p.m);
    } else {
      stage_x<XT, kHasLo, kCorrStride, true, 4>(static_cast<const XT*>(o.x), p.m, o.k, 0, o.k >> 5, xs, kXsStride, corr);
    }
    __syncthreads();
    trace_stamp(p, op, kTraceStaged);

    const uint32_t slabs = o.slabs, rounds = o.rounds;
    for (uint32_t round = 0; round < rounds; ++round) {
      const PairItem it = round == 0 ? first_item : pair_item_of<kCB>(o, round, warp, grid, cta);
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int j = 0; j < kAcc; ++j) acc[r][j] = 0.0f;
      // (1) the bias of the rows this lane will store, fetched while the weights are consumed
      const uint32_t local_row = (it.rb - o.rb_begin[it.wi]) * 16u;  // first row of the pair inside its weight
      float bias_pre[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      if (it.valid) {
        const float* bias = o.bias[it.wi];
        const float* bias2 = (o.flags & kOpSwiglu) ? o.bias[1] : bias + 16;  // bias of the pair's second block
        if (o.slabs == 1) {
          bias_pre[0] = bias[local_row + g];
          bias_pre[1] = bias[local_row + g + 8];
          bias_pre[2] = bias2[local_row + g];
          bias_pre[3] = bias2[local_row + g + 8];
        } else if (!(o.flags & kOpSwiglu)) {
          bias_pre[0] = bias[local_row + lane];  // the reducer's first pass covers rows lane of the pair
          // ... and so does its residual (one activation row: output index == row)
          if (p.m == 1 && o.residual[it.wi] != nullptr) bias_pre[1] = o.residual[it.wi][local_row + lane];
        }
      }

      for (uint32_t first = 0; first < it.nck; first += kPiece) {
        const uint32_t nc = min(static_cast<uint32_t>(kPiece), it.nck - first);
        const uint32_t slot = cons_q & (kNS - 1), parity = (cons_q / kNS) & 1u;
        {
          uint32_t spins = 0;
          while (!mbar_try_wait(bars + slot * 8, parity)) {
            if (++spins > kSpinLimit) {
              *reinterpret_cast<volatile int*>(p.status) = 2;
              break;
            }
          }
        }
        if (first == 0 && round == 0) trace_stamp(p, op, kTraceFirstPiece);
        const uint32_t slot_addr = ring + slot * kSlotBytes;
        const uint32_t unit0 = (it.c0 + first) / kCU;
        const uint32_t w_base = slot_addr + lane * 16, s_base = slot_addr + scale_lane;
        const uint32_t xs_base = xs_lane + unit0 * 512, corr_base = corr_lane + unit0 * (kG * kCorrStride * 8);
        if (nc == kPiece) {
          static_for<kPieceUnits>([&](auto ku) { unit_step(ku, w_base, s_base, xs_base, corr_base); });
        } else {
          for (uint32_t u = 0; u * kCU < nc; ++u)
            unit_step(std::integral_constant<int, 0>{}, w_base + u * (kCU * kCB), s_base + u * (kCU * kCB),
                      xs_base + u * 512, corr_base + u * (kG * kCorrStride * 8));
        }
        __syncwarp();  // every lane has read the slot: it can take the next piece
        produce();
        cons_q += 1;
      }

      // ---- this round's outputs ------------------------------------------------------
      if (round == 0) trace_stamp(p, op, kTraceConsumed);
      // lanes whose C columns belong to different groups hold partial sums of the same outputs
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int j = 0; j < kAcc; ++j) {
          if constexpr (kG == 4) acc[r][j] += __shfl_xor_sync(0xffffffffu, acc[r][j], 1);
          acc[r][j] += __shfl_xor_sync(0xffffffffu, acc[r][j], 2);
        }
      const bool owner = jl == 0;
      // Ops with a SiLU gate, a residual or a cross-rank reduce finish in functions of their own
      // (not inlined: their registers must not weigh on the loop above); plain ops store here.
      const bool plain = o.flags == 0 && o.residual[it.wi] == nullptr;
      if (slabs == 1) {
        if (it.nck != 0 && owner) {
#pragma unroll
          for (int j = 0; j < (kHasLo ? 1 : 2); ++j) {
            const uint32_t mm = kHasLo ? tl : 2 * tl + j;
            if (mm >= p.m) continue;
            const float a0 = acc[0][kHasLo ? 0 : j], a1 = acc[0][kHasLo ? 1 : 2 + j];
            const float b0 = acc[1][kHasLo ? 0 : j], b1 = acc[1][kHasLo ? 1 : 2 + j];
            if (plain) {
              float* dst = o.out[it.wi] + static_cast<size_t>(mm) * o.n[it.wi] + local_row + g;
              dst[0] = fmaf(a0, kUnscale, bias_pre[0]);
              dst[8] = fmaf(a1, kUnscale, bias_pre[1]);
              dst[16] = fmaf(b0, kUnscale, bias_pre[2]);
              dst[24] = fmaf(b1, kUnscale, bias_pre[3]);
            } else {
              finish_fused_lane(&o, it.wi, mm, local_row + g, a0, a1, b0, b1, bias_pre[0], bias_pre[1], bias_pre[2],
                                bias_pre[3], p.fcomm, p.status);
            }
          }
        }
        continue;
      }
      // K was split over `slabs` warps of this CTA: meet in shared memory, add in slab order.
      float* mine = red + (static_cast<size_t>(red_buf) * kPlanWarps + warp) * (2 * p.m * 16);
      if (owner) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int j = 0; j < (kHasLo ? 1 : 2); ++j) {
            const uint32_t mm = kHasLo ? tl : 2 * tl + j;
            if (mm >= p.m) continue;
            mine[(r * p.m + mm) * 16 + g] = acc[r][kHasLo ? 0 : j];  // zeros when the warp had no chunks
            mine[(r * p.m + mm) * 16 + g + 8] = acc[r][kHasLo ? 1 : 2 + j];
          }
      }
      __syncthreads();
      if ((warp & (slabs - 1u)) == 0 && it.valid) {
        const float* first_slab = mine;
        if (plain) {
          const uint32_t n_i = o.n[it.wi];
          float* out = o.out[it.wi];
          const float* bias = o.bias[it.wi];
          for (uint32_t idx = lane; idx < 32u * p.m; idx += 32) {
            float total = 0.0f;
            for (uint32_t sl = 0; sl < slabs; ++sl) total += first_slab[static_cast<size_t>(sl) * (2 * p.m * 16) + idx];
            const uint32_t r = idx / (p.m * 16), rem = idx - r * (p.m * 16);
            const uint32_t mm = rem >> 4, row = local_row + r * 16 + (rem & 15u);
            // idx == lane in the first pass: row r * 16 + (lane & 15) of activation row 0 when m == 1
            const float b = (idx == lane && p.m == 1) ? bias_pre[0] : bias[row];
            out[static_cast<size_t>(mm) * n_i + row] = fmaf(total, kUnscale, b);
          }
        } else {
          finish_fused_slabs(&o, it.wi, first_slab, slabs, p.m, local_row, lane, bias_pre[0], bias_pre[1], p.fcomm, p.status);
        }
      }
      red_buf ^= 1u;  // the next round writes the other buffer; this one is re-used two rounds on
    }
    trace_stamp(p, op, kTraceOpEnd);
  }
  if (p.fcomm != nullptr && p.reduce_ops != 0) {
    // the last CTA to get here advances the epoch for the next launch
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const unsigned int finished = atomicAdd(p.fcomm->done, 1u) + 1u;
      if (finished == gridDim.x) {
        *reinterpret_cast<volatile unsigned int*>(p.fcomm->done) = 0u;
        __threadfence();
        // (nobody writes the epoch before this point, so it still holds the launch's base)
        const unsigned int epoch_base = *reinterpret_cast<volatile unsigned int*>(p.fcomm->epoch);
        *reinterpret_cast<volatile unsigned int*>(p.fcomm->epoch) = epoch_base + p.reduce_ops;
      }
    }
  }
}

}  // namespace

// ---- host side ------------------------------------------------------------------------

struct PlanCopy {
  bool to_device;
  void* device;
  void* host;
  uint64_t bytes;
};

struct Plan {
  std::vector<PlanOpDev> ops;
  std::vector<PlanCopy> before, after;
  PlanOpDev* ops_dev = nullptr;
  unsigned int* grid_bar = nullptr;
  int* status_host = nullptr;  // mapped
  int* status_dev = nullptr;
  uint32_t m = 0;
  int x_dtype = 0;
  int scale_dtype = 0;
  uint32_t k_max = 0;
  bool all_even_chunks = true;  // every op's k is a multiple of 128
  bool all_even_blocks = true;  // every weight has a whole number of 32-row pairs
  bool any_fused = false;       // some op carries a norm, a SiLU gate, a residual or a cross-rank reduce
  uint32_t reduce_ops = 0;      // kOpReduce ops recorded
  const FusedCommDev* fcomm = nullptr;
  bool paired = false;          // plan_pair_kernel: work items are pairs of row blocks
  uint32_t unit_chunks = 1;     // chunks the kernel consumes at a time (slabs are whole units)
  int grid = 0;
  size_t smem = 0;
  uint32_t xs_bytes = 0;
  void* kernel = nullptr;
};

namespace {

constexpr size_t kSmemBudget = 227 * 1024;

template <typename XT, bool kScaleF16, int kCols, int kSlotChunks, int kG>
cudaError_t configure(Plan& plan, int sm_count, bool* fits) {
  auto kernel = plan_kernel<XT, kScaleF16, kCols, kSlotChunks, kG>;
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kCpg = 8 / kG;
  const uint32_t cb = kChunkWeightBytes + 32u * (kScaleF16 ? 2u : 4u);
  const uint32_t active_cols = kHasLo ? 2 * plan.m : plan.m;
  const uint32_t groups = plan.k_max / 32;
  const size_t xs_bytes = static_cast<size_t>(groups) * (kG > 1 ? kCpg : active_cols) * 64;
  const uint32_t corr_stride = kG > 1 ? (kHasLo ? kCpg / 2 : kCpg) : (kHasLo ? kCols / 2 : kCols);
  const size_t smem = static_cast<size_t>(kPlanWarps) * kSlots * kSlotChunks * cb + kPlanWarps * kSlots * 8 + xs_bytes +
                      static_cast<size_t>(groups) * corr_stride * 8 +
                      static_cast<size_t>(2) * kPlanWarps * plan.m * 16 * sizeof(float);
  plan.unit_chunks = kG > 1 ? kG / 2 : 1;
  *fits = smem <= kSmemBudget;
  if (!*fits) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kPlanWarps * 32, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  plan.kernel = reinterpret_cast<void*>(kernel);
  plan.smem = smem;
  plan.xs_bytes = static_cast<uint32_t>(xs_bytes);
  plan.grid = sm_count;  // one CTA per SM; all co-resident (cooperative launch)
  return cudaSuccess;
}

template <typename XT, bool kScaleF16, int kG, int kPiece, int kNS>
cudaError_t configure_pair(Plan& plan, int sm_count, bool* fits) {
  static_assert((kNS & (kNS - 1)) == 0, "the slot of a piece is its sequence number modulo a power of two");
  auto kernel = plan_pair_kernel<XT, kScaleF16, kG, kPiece, kNS>;
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kCpg = 8 / kG;
  const uint32_t cb = kChunkWeightBytes + 32u * (kScaleF16 ? 2u : 4u);
  const uint32_t groups = plan.k_max / 32;
  const size_t xs_bytes = static_cast<size_t>(groups) * kCpg * 64;
  const size_t smem = static_cast<size_t>(kPlanWarps) * kNS * 2 * kPiece * cb + kPlanWarps * kNS * 8 + xs_bytes +
                      static_cast<size_t>(groups) * (kHasLo ? kCpg / 2 : kCpg) * 8 +
                      static_cast<size_t>(2) * kPlanWarps * 2 * plan.m * 16 * sizeof(float) + 16 +
                      kOpWindow * sizeof(PlanOpDev);
  *fits = smem <= kSmemBudget;
  if (!*fits) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kPlanWarps * 32, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  plan.kernel = reinterpret_cast<void*>(kernel);
  plan.smem = smem;
  plan.xs_bytes = static_cast<uint32_t>(xs_bytes);
  plan.grid = sm_count;
  plan.unit_chunks = kG / 2;
  plan.paired = true;
  return cudaSuccess;
}

template <typename XT, bool kScaleF16, int kG>
cudaError_t configure_pair_slots(Plan& plan, int sm_count, bool* fits) {
  // Four slots of two chunks time the same as two slots of four (measured): what counts is the
  // number of bytes a warp keeps in flight, and shared memory bounds that.
  cudaError_t e = configure_pair<XT, kScaleF16, kG, 4, 2>(plan, sm_count, fits);
  if (e != cudaSuccess || *fits) return e;
  return configure_pair<XT, kScaleF16, kG, 2, 2>(plan, sm_count, fits);
}

// Deep weight rings when the staged activations leave room for them, shallower ones otherwise.
template <typename XT, bool kScaleF16, int kCols, int kG>
cudaError_t configure_slots(Plan& plan, int sm_count, bool* fits) {
  cudaError_t e = configure<XT, kScaleF16, kCols, 8, kG>(plan, sm_count, fits);
  if (e != cudaSuccess || *fits) return e;
  return configure<XT, kScaleF16, kCols, 4, kG>(plan, sm_count, fits);
}

template <typename XT>
cudaError_t configure_x(Plan& plan, int sm_count, bool* fits) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  const bool f16s = plan.scale_dtype == KQ_F16;
  const uint32_t cols = kHasLo ? 2 * plan.m : plan.m;
  // Few columns: several scale groups share one MMA tile (four need whole pairs of chunks);
  // with whole 32-row pairs everywhere, the paired kernel.
  if (plan.all_even_blocks && cols <= 4) {
    cudaError_t e;
    if (cols <= 2 && plan.all_even_chunks)
      e = f16s ? configure_pair_slots<XT, true, 4>(plan, sm_count, fits) : configure_pair_slots<XT, false, 4>(plan, sm_count, fits);
    else
      e = f16s ? configure_pair_slots<XT, true, 2>(plan, sm_count, fits) : configure_pair_slots<XT, false, 2>(plan, sm_count, fits);
    if (e != cudaSuccess || *fits) return e;
  }
  if (cols <= 2 && plan.all_even_chunks)
    return f16s ? configure_slots<XT, true, 8, 4>(plan, sm_count, fits) : configure_slots<XT, false, 8, 4>(plan, sm_count, fits);
  if (cols <= 4)
    return f16s ? configure_slots<XT, true, 8, 2>(plan, sm_count, fits) : configure_slots<XT, false, 8, 2>(plan, sm_count, fits);
  if (cols <= 8)
    return f16s ? configure_slots<XT, true, 8, 1>(plan, sm_count, fits) : configure_slots<XT, false, 8, 1>(plan, sm_count, fits);
  if (cols <= 16)
    return f16s ? configure_slots<XT, true, 16, 1>(plan, sm_count, fits) : configure_slots<XT, false, 16, 1>(plan, sm_count, fits);
  if constexpr (kHasLo) {
    return f16s ? configure_slots<XT, true, 32, 1>(plan, sm_count, fits) : configure_slots<XT, false, 32, 1>(plan, sm_count, fits);
  } else {
    return cudaErrorInvalidValue;
  }
}

cudaError_t configure_any(Plan& plan, int sm_count, bool* fits) {
  switch (plan.x_dtype) {
    case KQ_F32: return configure_x<float>(plan, sm_count, fits);
    case KQ_F16: return configure_x<__half>(plan, sm_count, fits);
    case KQ_BF16: return configure_x<__nv_bfloat16>(plan, sm_count, fits);
    default: return cudaErrorInvalidValue;
  }
}

// How an op is cut once the grid size is known: split K over S warps of a CTA until the
// op offers work to most of the grid; a pure function of the shape.
void shape_op(PlanOpDev& o, uint32_t grid, uint32_t unit_chunks, bool paired, uint32_t* rot) {
  uint32_t s = 1, log2 = 0;
  const uint32_t units_per_row = o.chunks_per_row / unit_chunks;
  // what one warp works on per round: a row block, a pair of adjacent ones, or (SiLU gate) the
  // same block of the gate and of the up weight
  const uint32_t items = !paired ? o.row_blocks : ((o.flags & kOpSwiglu) ? o.row_blocks : o.row_blocks / 2);
  while (s < static_cast<uint32_t>(kPlanWarps) && s * 2 <= units_per_row &&
         (items + kPlanWarps / s - 1) / (kPlanWarps / s) < (grid * 3) / 5) {
    s *= 2;
    ++log2;
  }
  o.slabs = s;
  o.slabs_log2 = log2;
  o.chunks_per_slab = (units_per_row + s - 1) / s * unit_chunks;
  o.cta_items = (items + kPlanWarps / s - 1) / (kPlanWarps / s);
  o.rounds = (o.cta_items + grid - 1) / grid;
  o.rot = *rot;
  *rot = (*rot + o.cta_items) % grid;  // the next op starts where this one left the grid idle
}

bool fill_op(PlanOpDev& o, int count, const LinearTarget* targets, const void* x, const LinearFusion& fusion,
             const char** why) {
  o = PlanOpDev{};
  o.count = static_cast<uint32_t>(count);
  const Weight& w0 = *targets[0].w;
  if (fusion.swiglu) {
    if (count != 2 || targets[0].w->n != targets[1].w->n) {
      *why = "the SiLU gate takes exactly two weights (gate, up) with the same number of rows";
      return false;
    }
    if (fusion.reduce || fusion.residual != nullptr) {
      *why = "the SiLU gate combines with a norm only";
      return false;
    }
    o.gate_up_delta = static_cast<const uint8_t*>(targets[1].w->data) - static_cast<const uint8_t*>(targets[0].w->data);
    o.flags |= kOpSwiglu;
  }
  if (fusion.reduce || fusion.residual != nullptr) {
    if (count != 1) {
      *why = "a residual or a cross-rank reduce goes with a single weight";
      return false;
    }
    if (fusion.reduce) o.flags |= kOpReduce;
  }
  o.norm_weight = fusion.norm_weight;
  o.norm_eps = fusion.norm_eps;
  uint32_t rb = 0;
  for (int i = 0; i < count; ++i) {
    const Weight& w = *targets[i].w;
    if (w.layout != kLayoutTiledI4) {
      *why = "a weight is not in the tiled int4 / group-32 layout";
      return false;
    }
    if (w.k != w0.k || w.scale_dtype != w0.scale_dtype) {
      *why = "weights of one op differ in k or scale type";
      return false;
    }
    o.w[i] = static_cast<const uint8_t*>(w.data);
    o.bias[i] = targets[i].bias;
    o.out[i] = targets[i].out;
    o.residual[i] = i == 0 ? fusion.residual : nullptr;
    o.n[i] = w.n;
    o.rb_begin[i] = rb;
    rb += w.n / 16;
  }
  if (fusion.swiglu) rb = w0.n / 16;  // items are counted in blocks of ONE of the two weights
  for (int i = count; i <= kMaxMulti; ++i) o.rb_begin[i] = rb;
  o.x = x;
  o.k = w0.k;
  o.chunks_per_row = w0.k / kChunkK;
  o.row_blocks = rb;
  return true;
}

}  // namespace

Plan* plan_create() { return new Plan(); }

void plan_destroy(Plan* plan) {
  if (!plan) return;
  if (plan->ops_dev) cudaFree(plan->ops_dev);
  if (plan->grid_bar) cudaFree(plan->grid_bar);
  if (plan->status_host) cudaFreeHost(plan->status_host);
  delete plan;
}

// Host-to-device copies run before the kernel and device-to-host copies after it, so a write
// recorded after the first linear or a read recorded before it cannot keep its place in the
// recorded order: both are refused (the plan then fails to finalize) rather than replayed
// somewhere else.  Returns an empty string when the copy was recorded.
const char* plan_add_copy(Plan* plan, bool to_device, void* device, void* host, uint64_t bytes) {
  if (to_device) {
    if (!plan->ops.empty()) return "a host write was recorded after a linear; writes must come before the first op";
    plan->before.push_back(PlanCopy{true, device, host, bytes});
  } else {
    if (plan->ops.empty()) return "a host read was recorded before any linear; reads must come after the last op";
    plan->after.push_back(PlanCopy{false, device, host, bytes});
  }
  return "";
}

// Returns an empty string when the op was recorded, else why the fused kernel cannot run it.
const char* plan_add_linear(Plan* plan, int count, const LinearTarget* targets, const void* x, int x_dtype,
                            uint32_t m, const LinearFusion& fusion) {
  if (!plan->after.empty()) return "a host read was recorded before this linear; reads must come after the last op";
  if (m < 1 || m > 16) return "the fused plan kernel covers 1..16 activation rows";
  if (count < 1 || count > kMaxMulti) return "too many weights in one op";
  PlanOpDev o;
  const char* why = "";
  if (!fill_op(o, count, targets, x, fusion, &why)) return why;
  if (o.flags & kOpReduce) {
    if (static_cast<uint64_t>(m) * o.n[0] * 8u > kFusedSlotBytes)
      return "a cross-rank reduce inside a plan exchanges at most 8192 outputs per op";
    o.reduce_index = plan->reduce_ops;
    plan->reduce_ops += 1;
  }
  if (o.flags != 0 || o.norm_weight != nullptr || o.residual[0] != nullptr) plan->any_fused = true;
  const int scale_dtype = targets[0].w->scale_dtype;
  if (plan->ops.empty()) {
    plan->m = m;
    plan->x_dtype = x_dtype;
    plan->scale_dtype = scale_dtype;
  } else if (plan->m != m || plan->x_dtype != x_dtype || plan->scale_dtype != scale_dtype) {
    return "ops of one plan must share m, the activation type and the scale type";
  }
  plan->k_max = std::max(plan->k_max, o.k);
  plan->all_even_chunks = plan->all_even_chunks && o.chunks_per_row % 2 == 0;
  if (!(o.flags & kOpSwiglu))
    for (int i = 0; i < count; ++i) plan->all_even_blocks = plan->all_even_blocks && targets[i].w->n % 32 == 0;
  plan->ops.push_back(o);
  return "";
}

uint32_t plan_op_count(const Plan* plan) { return static_cast<uint32_t>(plan->ops.size()); }
uint32_t plan_grid(const Plan* plan) { return static_cast<uint32_t>(plan->grid); }
bool plan_is_paired(const Plan* plan) { return plan->paired; }
uint32_t plan_trace_slots() { return kTraceSlots; }

cudaError_t plan_finalize(Plan* plan, const LaunchEnv& env, const char** why) {
  *why = "";
  if (plan->ops.empty()) {
    *why = "the plan holds no linear op";
    return cudaErrorInvalidValue;
  }
  bool fits = false;
  cudaError_t e = configure_any(*plan, env.sm_count, &fits);
  if (e != cudaSuccess) return e;
  if (!fits) {
    *why = "the staged activations of the widest op (k * columns * 2 bytes) do not fit in shared memory next to the weight rings";
    return cudaErrorInvalidValue;
  }
  if (plan->any_fused && !plan->paired) {
    *why = "ops with a norm, a SiLU gate, a residual or a cross-rank reduce need the paired kernel: at most two "
           "f32 / bf16 rows (four binary16 rows) and weights with a whole number of 32-row pairs";
    return cudaErrorInvalidValue;
  }
  if (plan->reduce_ops != 0) {
    if (env.fused == nullptr) {
      *why = "the plan holds a cross-rank reduce but the context has no connected exchange (kq_comm_connect)";
      return cudaErrorInvalidValue;
    }
    plan->fcomm = env.fused;
  }
  uint32_t rot = 0;
  for (PlanOpDev& o : plan->ops) shape_op(o, static_cast<uint32_t>(plan->grid), plan->unit_chunks, plan->paired, &rot);
  e = cudaMalloc(reinterpret_cast<void**>(&plan->ops_dev), plan->ops.size() * sizeof(PlanOpDev));
  if (e == cudaSuccess) e = cudaMemcpy(plan->ops_dev, plan->ops.data(), plan->ops.size() * sizeof(PlanOpDev), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&plan->grid_bar), sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&plan->status_host), sizeof(int), cudaHostAllocMapped);
  if (e == cudaSuccess) {
    *plan->status_host = 0;
    e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&plan->status_dev), plan->status_host, 0);
  }
  return e;
}

cudaError_t plan_launch(Plan* plan, const LaunchEnv& env, int* launches, unsigned long long* trace) {
  cudaError_t e = cudaSuccess;
  for (const PlanCopy& c : plan->before) {
    e = cudaMemcpyAsync(c.device, c.host, c.bytes, cudaMemcpyHostToDevice, env.stream);
    if (e != cudaSuccess) return e;
  }
  e = cudaMemsetAsync(plan->grid_bar, 0, sizeof(unsigned int), env.stream);
  if (e != cudaSuccess) return e;
  PlanParams p = {};
  p.ops = plan->ops_dev;
  p.op_count = static_cast<uint32_t>(plan->ops.size());
  p.m = plan->m;
  p.xs_bytes = plan->xs_bytes;
  p.grid_bar = plan->grid_bar;
  p.status = plan->status_dev;
  p.fcomm = plan->fcomm;
  p.reduce_ops = plan->reduce_ops;
  p.trace = plan->paired ? trace : nullptr;  // the paired kernel is the one that leaves stamps
  void* args[] = {&p};
  e = cudaLaunchCooperativeKernel(plan->kernel, dim3(plan->grid), dim3(kPlanWarps * 32), args, plan->smem, env.stream);
  if (e != cudaSuccess) return e;
  if (launches) *launches += 1;
  for (const PlanCopy& c : plan->after) {
    e = cudaMemcpyAsync(c.host, c.device, c.bytes, cudaMemcpyDeviceToHost, env.stream);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

int plan_take_status(Plan* plan) {
  const int s = *reinterpret_cast<volatile int*>(plan->status_host);
  *reinterpret_cast<volatile int*>(plan->status_host) = 0;
  return s;
}

// ---- one linear, no allocation -------------------------------------------------------
// Everything the fused kernel needs in global memory besides the caller's tensors lives
// in one file-scope device array that every GPU loading this library carries until the
// process exits:
//   [0, 256)      grid-barrier word
//   [256, 512)    status word
//   [512, 1024)   the op descriptor
constexpr size_t kStaticBarOff = 0;
constexpr size_t kStaticStatusOff = 256;
constexpr size_t kStaticOpOff = 512;
constexpr size_t kStaticTotal = 4096;
static_assert(sizeof(PlanOpDev) <= 512 && sizeof(PlanOpDev) % 4 == 0, "op descriptor outgrew its slot");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticTotal];

constexpr int kStaticMaxDevices = 64;
static unsigned char* g_static_base[kStaticMaxDevices] = {};  // device address of the array, per device

// In host code `g_static_scratch` is only a handle: the address a kernel may use comes
// from cudaGetSymbolAddress, asked once per device with that device current.
static cudaError_t static_scratch_for_current_device(unsigned char** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kStaticMaxDevices) return cudaErrorInvalidDevice;
  if (!g_static_base[device]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return e;
    e = cudaMemset(ptr, 0, kStaticTotal);
    if (e != cudaSuccess) return e;
    g_static_base[device] = static_cast<unsigned char*>(ptr);
  }
  *out = g_static_base[device];
  return cudaSuccess;
}

cudaError_t linear_static(const LaunchEnv& env, const LinearTarget& target, const void* x, int x_dtype,
                          uint32_t m, const char** why, int* device_status) {
  *why = "";
  *device_status = 0;
  if (m < 1 || m > 16) {
    *why = "1..16 activation rows";
    return cudaErrorInvalidValue;
  }
  PlanOpDev o;
  if (!fill_op(o, 1, &target, x, LinearFusion{}, why)) return cudaErrorInvalidValue;
  unsigned char* base = nullptr;
  cudaError_t e = static_scratch_for_current_device(&base);
  if (e != cudaSuccess) return e;

  Plan cfg;  // only carries the kernel choice; its vectors stay empty (no heap use)
  cfg.m = m;
  cfg.x_dtype = x_dtype;
  cfg.scale_dtype = target.w->scale_dtype;
  cfg.k_max = o.k;
  cfg.all_even_chunks = o.chunks_per_row % 2 == 0;
  cfg.all_even_blocks = target.w->n % 32 == 0;
  bool fits = false;
  e = configure_any(cfg, env.sm_count, &fits);
  if (e != cudaSuccess) return e;
  if (!fits) {
    *why = "k * columns * 2 bytes of staged activations exceed the kernel's shared-memory budget "
           "(columns = m for binary16 activations, 2 m for f32 / bf16)";
    return cudaErrorInvalidValue;
  }
  uint32_t rot = 0;
  shape_op(o, static_cast<uint32_t>(cfg.grid), cfg.unit_chunks, cfg.paired, &rot);

  e = cudaMemcpyAsync(base + kStaticOpOff, &o, sizeof(o), cudaMemcpyHostToDevice, env.stream);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(base + kStaticBarOff, 0, 512, env.stream);  // barrier word and status word
  if (e != cudaSuccess) return e;
  PlanParams p = {};
  p.ops = reinterpret_cast<const PlanOpDev*>(base + kStaticOpOff);
  p.op_count = 1;
  p.m = m;
  p.xs_bytes = cfg.xs_bytes;
  p.grid_bar = reinterpret_cast<unsigned int*>(base + kStaticBarOff);
  p.status = reinterpret_cast<int*>(base + kStaticStatusOff);
  void* args[] = {&p};
  e = cudaLaunchCooperativeKernel(cfg.kernel, dim3(cfg.grid), dim3(kPlanWarps * 32), args, cfg.smem, env.stream);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyAsync(device_status, base + kStaticStatusOff, sizeof(int), cudaMemcpyDeviceToHost, env.stream);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(env.stream);
}

}  // namespace kq
