// kq_plan — a recorded sequence of quantized linears executed by ONE persistent kernel.
//
// Replaces the reference's baked-plan replay (executeBakedPlan,
// packages/runtime/src/runtime/recipe.ts:462) for plans made of int4 / group-32 linears with
// at most 16 activation rows — a decode step.  Launching those ~130 small, dependent
// matmuls one by one costs more in launch and drain latency than in memory time; here one
// CTA per SM stays resident for the whole plan and the weight stream never stops:
//
//   * every warp owns a static, interleaved list of work items (16 output channels x 512 k
//     = 4.6 KB of the tiled layout) across ALL ops of the plan, and keeps two of them in
//     flight in its private shared-memory ring with cp.async.bulk + mbarrier.  The copies
//     for the next op are issued before the warp waits for the previous op to finish, so
//     HBM keeps streaming through the dependency barriers;
//   * the math per 64-k chunk is the same as in qgemv_i4_kernel (kq_gemv_core.cuh): nibble
//     pairs as binary16 subnormals into mma.sync, hi/lo activation columns, f32 group scale;
//   * partial sums of the k-slabs of one 16-row block meet in the context workspace; the
//     warp that delivers the last slab adds them in slab order (deterministic) and writes
//     the output row block;
//   * ops are separated by a grid-wide barrier (all CTAs are co-resident: cooperative
//     launch).  Every wait in this file is bounded: if one gives up, the kernel records a
//     status word, keeps going without blocking, and the host reports KQ_ERR_TIMEOUT.
#include <algorithm>
#include <type_traits>
#include <vector>

#include "kq_gemv_core.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kPlanWarps = 16;
constexpr int kSlotChunks = 8;  // chunks (64 k each) per work item = per ring slot
constexpr int kSlots = 2;       // ring slots per warp
constexpr uint32_t kSpinLimit = 1u << 22;

struct PlanOpDev {
  const uint8_t* w[kMaxMulti];
  const float* bias[kMaxMulti];
  float* out[kMaxMulti];
  uint32_t n[kMaxMulti];
  uint32_t rb_begin[kMaxMulti + 1];  // prefix sums of n / 16
  uint32_t count;
  const void* x;
  uint32_t k;
  uint32_t chunks_per_row;  // k / 64
  uint32_t slabs;           // k-slabs of kSlotChunks chunks per row block
  uint32_t row_blocks;      // total 16-row blocks of the op
  uint32_t row_blocks_padded;  // rounded up to kPlanWarps: all items of a CTA round share a slab
  uint32_t items;           // slabs * row_blocks_padded
  uint32_t n_total;
};

struct PlanParams {
  const PlanOpDev* ops;
  uint32_t op_count;
  uint32_t m;
  float* partial;          // [slab][m][n_total] of the op being executed
  unsigned int* counters;  // per 16-row block: slabs delivered (self-resetting)
  unsigned int* grid_bar;  // arrivals at the inter-op barrier (zeroed before every launch)
  int* error_flag;         // activation out of domain
  int* status;             // non-zero: a bounded wait gave up
};

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

// Position of a warp in its list of work items.
struct ItemCursor {
  uint32_t op, round;
};

template <typename XT, bool kScaleF16, int kCols>
__global__ void __launch_bounds__(kPlanWarps * 32, 1)
plan_kernel(const PlanParams p) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;  // chunk bytes
  constexpr uint32_t kSlotBytes = kSlotChunks * kCB;
  constexpr int kTiles = kCols / 8;
  constexpr int kAccPerTile = kHasLo ? 2 : 4;
  constexpr int kCorrPerTile = kHasLo ? 1 : 2;
  constexpr int kCorrStride = kHasLo ? kCols / 2 : kCols;
  constexpr uint32_t kMask0 = 0x000F000Fu, kMask1 = 0x00F000F0u;

  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t gw = blockIdx.x * kPlanWarps + warp;  // this warp's index in the grid
  const uint32_t GW = gridDim.x * kPlanWarps;

  // shared memory: [warp rings][mbarriers][x slab][corr]
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t ring = smem_base + warp * (kSlots * kSlotBytes);
  const uint32_t bars = smem_base + kPlanWarps * kSlots * kSlotBytes + warp * (kSlots * 8);
  uint8_t* xs = smem + kPlanWarps * kSlots * kSlotBytes + kPlanWarps * kSlots * 8;
  const uint32_t active_cols = kHasLo ? 2 * p.m : p.m;
  const uint32_t xs_stride = active_cols * 64;
  float* corr = reinterpret_cast<float*>(xs + 2 * kSlotChunks * xs_stride);

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kSlots; ++s) mbar_init(bars + s * 8, 1);
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  // Decodes work item `item` of op `o`; false for the padding items of a slab.
  auto locate = [&](const PlanOpDev& o, uint32_t item, const uint8_t*& src, uint32_t& nck, uint32_t& rb,
                    uint32_t& ks, uint32_t& wi) -> bool {
    ks = item / o.row_blocks_padded;
    rb = item - ks * o.row_blocks_padded;
    if (rb >= o.row_blocks) return false;
    wi = 0;
#pragma unroll
    for (int i = 1; i < kMaxMulti; ++i)
      if (i < static_cast<int>(o.count) && rb >= o.rb_begin[i]) wi = i;
    const uint32_t c0 = ks * kSlotChunks;
    nck = min(static_cast<uint32_t>(kSlotChunks), o.chunks_per_row - c0);
    src = o.w[wi] + (static_cast<size_t>(rb - o.rb_begin[wi]) * o.chunks_per_row + c0) * kCB;
    return true;
  };

  // Producer side: start the copy of this warp's next work item (whatever op it belongs
  // to) into the ring slot that sequence number prod_q maps to.
  ItemCursor prod{0, 0};
  uint32_t prod_q = 0;
  auto produce = [&]() {
    while (prod.op < p.op_count) {
      const PlanOpDev& o = p.ops[prod.op];
      const uint32_t item = prod.round * GW + gw;
      if (item >= o.items) {
        prod.op += 1;
        prod.round = 0;
        continue;
      }
      prod.round += 1;
      const uint8_t* src;
      uint32_t nck, rb, ks, wi;
      if (!locate(o, item, src, nck, rb, ks, wi)) continue;
      const uint32_t slot = prod_q & 1u;
      if (lane == 0) {
        mbar_expect_tx(bars + slot * 8, nck * kCB);
        bulk_copy_g2s(ring + slot * kSlotBytes, src, nck * kCB, bars + slot * 8);
      }
      prod_q += 1;
      return;
    }
  };
#pragma unroll
  for (int s = 0; s < kSlots; ++s) produce();

  // Persistent per-lane state of the MMA operands (see qgemv_i4_kernel).
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
      const uint32_t mm = kHasLo ? tile_m * 4 + t : tile_m * 8 + 2 * t + j;
      load_c[tile_m][j] = mm < p.m;
    }
  }
  const uint32_t xs_lane = static_cast<uint32_t>(__cvta_generic_to_shared(xs)) + lane * 16;
  const uint32_t corr_lane = static_cast<uint32_t>(__cvta_generic_to_shared(corr)) + (kHasLo ? t : 2 * t) * 4;

  uint32_t cons_q = 0;
  for (uint32_t op = 0; op < p.op_count; ++op) {
    const PlanOpDev& o = p.ops[op];
    if (op > 0) {
      // every output of the previous op must be complete and visible before x is read
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(p.grid_bar, 1u);
        const unsigned int target = op * gridDim.x;
        uint32_t spins = 0;
        while (ld_acquire_gpu(p.grid_bar) < target) {
          if (++spins > kSpinLimit) {
            *reinterpret_cast<volatile int*>(p.status) = 1;
            break;
          }
          __nanosleep(32);
        }
        __threadfence();
      }
      __syncthreads();
    }
    const XT* x = static_cast<const XT*>(o.x);
    const uint32_t rounds = (o.items + GW - 1) / GW;
    for (uint32_t round = 0; round < rounds; ++round) {
      const uint32_t base = round * GW + blockIdx.x * kPlanWarps;  // first item of this CTA
      if (base >= o.items) break;
      // the CTA's 16 items share one k-slab (row_blocks_padded is a multiple of 16)
      const uint32_t ks_cta = base / o.row_blocks_padded;
      const uint32_t c0 = ks_cta * kSlotChunks;
      const uint32_t nck_cta = min(static_cast<uint32_t>(kSlotChunks), o.chunks_per_row - c0);
      __syncthreads();  // the previous round's slab is no longer being read
      stage_x<XT, kHasLo, kCorrStride, true>(x, p.m, o.k, 2 * c0, 2 * nck_cta, xs, xs_stride, corr, p.error_flag);
      __syncthreads();

      const uint8_t* src;
      uint32_t nck, rb, ks, wi;
      const uint32_t item = base + warp;
      if (item >= o.items || !locate(o, item, src, nck, rb, ks, wi)) continue;

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
      float acc[kTiles][kAccPerTile];
#pragma unroll
      for (int i = 0; i < kTiles; ++i)
#pragma unroll
        for (int j = 0; j < kAccPerTile; ++j) acc[i][j] = 0.0f;

      const uint32_t slot_addr = ring + slot * kSlotBytes;
#pragma unroll 2
      for (uint32_t c = 0; c < nck; ++c) {
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
          const uint32_t lg = 2 * c + jj;
#pragma unroll
          for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
            lds_v4_if(bfrag[tile_m], xs_lane + lg * xs_stride + tile_m * 512, load_b[tile_m]);
#pragma unroll
            for (int j = 0; j < kCorrPerTile; ++j)
              lds_f32_if(cterm[tile_m][j], corr_lane + (lg * kCorrStride + tile_m * (kHasLo ? 4 : 8) + j) * 4,
                         load_c[tile_m][j]);
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
              acc[tile_m][0] = fmaf(s.x, (cf[0] + cf[1]) + cterm[tile_m][0], acc[tile_m][0]);
              acc[tile_m][1] = fmaf(s.y, (cf[2] + cf[3]) + cterm[tile_m][0], acc[tile_m][1]);
            } else {
              acc[tile_m][0] = fmaf(s.x, cf[0] + cterm[tile_m][0], acc[tile_m][0]);
              acc[tile_m][1] = fmaf(s.x, cf[1] + cterm[tile_m][1], acc[tile_m][1]);
              acc[tile_m][2] = fmaf(s.y, cf[2] + cterm[tile_m][0], acc[tile_m][2]);
              acc[tile_m][3] = fmaf(s.y, cf[3] + cterm[tile_m][1], acc[tile_m][3]);
            }
          }
        }
      }
      __syncwarp();  // every lane has read the slot: it can take the next item
      produce();
      cons_q += 1;

      // ---- this item's 16 rows x m partial sums ------------------------------------
      const uint32_t local_row = (rb - o.rb_begin[wi]) * 16u;  // first row of the block inside its weight
      const uint32_t n_i = o.n[wi];
      float* out = o.out[wi];
      const float* bias = o.bias[wi];
      const bool direct = o.slabs == 1;
#pragma unroll
      for (int tile_m = 0; tile_m < kTiles; ++tile_m) {
#pragma unroll
        for (int j = 0; j < (kHasLo ? 1 : 2); ++j) {
          const uint32_t mm = kHasLo ? tile_m * 4 + t : tile_m * 8 + 2 * t + j;
          if (mm >= p.m) continue;
          const float va = acc[tile_m][kHasLo ? 0 : j];
          const float vb = acc[tile_m][kHasLo ? 1 : 2 + j];
          if (direct) {
            out[static_cast<size_t>(mm) * n_i + local_row + g] = fmaf(va, kUnscale, bias[local_row + g]);
            out[static_cast<size_t>(mm) * n_i + local_row + g + 8] = fmaf(vb, kUnscale, bias[local_row + g + 8]);
          } else {
            float* part = p.partial + (static_cast<size_t>(ks) * p.m + mm) * o.n_total + rb * 16u + g;
            __stcg(part, va);
            __stcg(part + 8, vb);
          }
        }
      }
      if (direct) continue;
      // The warp that delivers the last k-slab of this row block adds all of them, in
      // slab order, and writes the block's outputs.
      __threadfence();
      __syncwarp();
      unsigned int arrived = 0;
      if (lane == 0) arrived = atomicAdd(p.counters + rb, 1u);
      arrived = __shfl_sync(0xffffffffu, arrived, 0);
      if (arrived != o.slabs - 1) continue;
      __threadfence();
      const size_t slab_stride = static_cast<size_t>(p.m) * o.n_total;
      for (uint32_t idx = lane; idx < 16u * p.m; idx += 32) {
        const uint32_t mm = idx >> 4, r = idx & 15u;
        const float* srcp = p.partial + static_cast<size_t>(mm) * o.n_total + rb * 16u + r;
        float total = 0.0f;
        uint32_t s = 0;
        for (; s + 4 <= o.slabs; s += 4) {
          const float v0 = __ldcg(srcp + (s + 0) * slab_stride), v1 = __ldcg(srcp + (s + 1) * slab_stride);
          const float v2 = __ldcg(srcp + (s + 2) * slab_stride), v3 = __ldcg(srcp + (s + 3) * slab_stride);
          total = (((total + v0) + v1) + v2) + v3;
        }
        for (; s < o.slabs; ++s) total += __ldcg(srcp + s * slab_stride);
        out[static_cast<size_t>(mm) * n_i + local_row + r] = fmaf(total, kUnscale, bias[local_row + r]);
      }
      if (lane == 0) p.counters[rb] = 0;  // ready for the next op / launch
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
  int grid = 0;
  size_t smem = 0;
  void* kernel = nullptr;
  uint64_t partial_bytes = 0;
  uint32_t max_row_blocks = 0;
};

namespace {

template <typename XT, bool kScaleF16, int kCols>
cudaError_t configure(Plan& plan, int sm_count) {
  auto kernel = plan_kernel<XT, kScaleF16, kCols>;
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  const uint32_t cb = kChunkWeightBytes + 32u * (kScaleF16 ? 2u : 4u);
  const uint32_t active_cols = kHasLo ? 2 * plan.m : plan.m;
  const size_t smem = static_cast<size_t>(kPlanWarps) * kSlots * kSlotChunks * cb + kPlanWarps * kSlots * 8 +
                      static_cast<size_t>(2 * kSlotChunks) * (active_cols * 64 + (kHasLo ? kCols / 2 : kCols) * 4);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kPlanWarps * 32, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  plan.kernel = reinterpret_cast<void*>(kernel);
  plan.smem = smem;
  plan.grid = sm_count;  // one CTA per SM; all co-resident (cooperative launch)
  return cudaSuccess;
}

template <typename XT>
cudaError_t configure_x(Plan& plan, int sm_count) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  const bool f16s = plan.scale_dtype == KQ_F16;
  const uint32_t cols = kHasLo ? 2 * plan.m : plan.m;
  if (cols <= 8) return f16s ? configure<XT, true, 8>(plan, sm_count) : configure<XT, false, 8>(plan, sm_count);
  if (cols <= 16) return f16s ? configure<XT, true, 16>(plan, sm_count) : configure<XT, false, 16>(plan, sm_count);
  if constexpr (kHasLo) {
    return f16s ? configure<XT, true, 32>(plan, sm_count) : configure<XT, false, 32>(plan, sm_count);
  } else {
    return cudaErrorInvalidValue;
  }
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

void plan_add_copy(Plan* plan, bool to_device, void* device, void* host, uint64_t bytes) {
  (plan->ops.empty() ? plan->before : plan->after).push_back(PlanCopy{to_device, device, host, bytes});
}

// Returns an empty string when the op was recorded, else why the fused kernel cannot run it.
const char* plan_add_linear(Plan* plan, int count, const LinearTarget* targets, const void* x, int x_dtype,
                            uint32_t m) {
  if (!plan->after.empty()) return "a host read was recorded before this linear; reads must come after the last op";
  if (m < 1 || m > 16) return "the fused plan kernel covers 1..16 activation rows";
  if (count < 1 || count > kMaxMulti) return "too many weights in one op";
  PlanOpDev o = {};
  o.count = static_cast<uint32_t>(count);
  const Weight& w0 = *targets[0].w;
  uint32_t rb = 0, n_total = 0;
  for (int i = 0; i < count; ++i) {
    const Weight& w = *targets[i].w;
    if (w.layout != kLayoutTiledI4) return "a weight is not in the tiled int4 / group-32 layout";
    if (w.k != w0.k || w.scale_dtype != w0.scale_dtype) return "weights of one op differ in k or scale type";
    o.w[i] = static_cast<const uint8_t*>(w.data);
    o.bias[i] = targets[i].bias;
    o.out[i] = targets[i].out;
    o.n[i] = w.n;
    o.rb_begin[i] = rb;
    rb += w.n / 16;
    n_total += w.n;
  }
  for (int i = count; i <= kMaxMulti; ++i) o.rb_begin[i] = rb;
  if (plan->ops.empty()) {
    plan->m = m;
    plan->x_dtype = x_dtype;
    plan->scale_dtype = w0.scale_dtype;
  } else if (plan->m != m || plan->x_dtype != x_dtype || plan->scale_dtype != w0.scale_dtype) {
    return "ops of one plan must share m, the activation type and the scale type";
  }
  o.x = x;
  o.k = w0.k;
  o.chunks_per_row = w0.k / kChunkK;
  o.slabs = (o.chunks_per_row + kSlotChunks - 1) / kSlotChunks;
  o.row_blocks = rb;
  o.row_blocks_padded = (rb + kPlanWarps - 1) / kPlanWarps * kPlanWarps;
  o.items = o.slabs * o.row_blocks_padded;
  o.n_total = n_total;
  plan->ops.push_back(o);
  if (o.slabs > 1)
    plan->partial_bytes = std::max<uint64_t>(plan->partial_bytes, static_cast<uint64_t>(o.slabs) * m * n_total * sizeof(float));
  plan->max_row_blocks = std::max(plan->max_row_blocks, rb);
  return "";
}

uint32_t plan_op_count(const Plan* plan) { return static_cast<uint32_t>(plan->ops.size()); }

cudaError_t plan_finalize(Plan* plan, const LaunchEnv& env, const char** why) {
  *why = "";
  if (plan->ops.empty()) {
    *why = "the plan holds no linear op";
    return cudaErrorInvalidValue;
  }
  if (plan->partial_bytes > env.workspace_bytes) {
    *why = "the plan's split-K partial sums do not fit the context workspace (raise workspace_bytes in kq_init)";
    return cudaErrorInvalidValue;
  }
  if (plan->max_row_blocks > env.counter_count) {
    *why = "an op has more 16-row blocks than the context has arrival counters";
    return cudaErrorInvalidValue;
  }
  cudaError_t e;
  switch (plan->x_dtype) {
    case KQ_F32: e = configure_x<float>(*plan, env.sm_count); break;
    case KQ_F16: e = configure_x<__half>(*plan, env.sm_count); break;
    case KQ_BF16: e = configure_x<__nv_bfloat16>(*plan, env.sm_count); break;
    default: return cudaErrorInvalidValue;
  }
  if (e != cudaSuccess) return e;
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

cudaError_t plan_launch(Plan* plan, const LaunchEnv& env, int* launches) {
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
  p.partial = static_cast<float*>(env.workspace);
  p.counters = env.counters;
  p.grid_bar = plan->grid_bar;
  p.error_flag = env.error_flag;
  p.status = plan->status_dev;
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
// Everything the fused kernel needs besides the caller's tensors lives in one file-scope
// device array that every GPU loading this library carries until the process exits:
//   [0, kStaticPartialBytes)        split-K partial sums
//   then kStaticCounters words      per-row-block arrival counters (kept at zero between calls)
//   then 256 B                      grid-barrier word
//   then 256 B                      status word
//   then 512 B                      the op descriptor
constexpr size_t kStaticPartialBytes = size_t(4) << 20;
constexpr uint32_t kStaticCounters = 8192;
constexpr size_t kStaticCountersOff = kStaticPartialBytes;
constexpr size_t kStaticBarOff = kStaticCountersOff + kStaticCounters * sizeof(unsigned int);
constexpr size_t kStaticStatusOff = kStaticBarOff + 256;
constexpr size_t kStaticOpOff = kStaticStatusOff + 256;
constexpr size_t kStaticTotal = kStaticOpOff + 512;
static_assert(sizeof(PlanOpDev) <= 512, "op descriptor outgrew its slot");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticTotal];

constexpr int kStaticMaxDevices = 64;
static unsigned char* g_static_base[kStaticMaxDevices] = {};  // device address of the array, per device

uint64_t linear_static_limit_bytes() { return kStaticPartialBytes; }

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
    // counters must start at zero (afterwards the kernel leaves them at zero itself)
    e = cudaMemset(static_cast<unsigned char*>(ptr) + kStaticCountersOff, 0,
                   kStaticCounters * sizeof(unsigned int));
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
  const Weight& w = *target.w;
  if (w.layout != kLayoutTiledI4) {
    *why = "the weight is not in the tiled int4 / group-32 layout";
    return cudaErrorInvalidValue;
  }
  if (m < 1 || m > 16) {
    *why = "1..16 activation rows";
    return cudaErrorInvalidValue;
  }
  PlanOpDev o = {};
  o.count = 1;
  o.w[0] = static_cast<const uint8_t*>(w.data);
  o.bias[0] = target.bias;
  o.out[0] = target.out;
  o.n[0] = w.n;
  o.rb_begin[0] = 0;
  for (int i = 1; i <= kMaxMulti; ++i) o.rb_begin[i] = w.n / 16;
  o.x = x;
  o.k = w.k;
  o.chunks_per_row = w.k / kChunkK;
  o.slabs = (o.chunks_per_row + kSlotChunks - 1) / kSlotChunks;
  o.row_blocks = w.n / 16;
  o.row_blocks_padded = (o.row_blocks + kPlanWarps - 1) / kPlanWarps * kPlanWarps;
  o.items = o.slabs * o.row_blocks_padded;
  o.n_total = w.n;
  if (o.slabs > 1 && static_cast<uint64_t>(o.slabs) * m * w.n * sizeof(float) > kStaticPartialBytes) {
    *why = "slabs * m * n * 4 bytes of partial sums exceed the 4 MiB static scratch";
    return cudaErrorInvalidValue;
  }
  if (o.row_blocks > kStaticCounters) {
    *why = "more than 8192 16-row blocks (n > 131072)";
    return cudaErrorInvalidValue;
  }
  unsigned char* base = nullptr;
  cudaError_t e = static_scratch_for_current_device(&base);
  if (e != cudaSuccess) return e;

  Plan cfg;  // only carries the kernel choice; its vectors stay empty (no heap use)
  cfg.m = m;
  cfg.x_dtype = x_dtype;
  cfg.scale_dtype = w.scale_dtype;
  switch (x_dtype) {
    case KQ_F32: e = configure_x<float>(cfg, env.sm_count); break;
    case KQ_F16: e = configure_x<__half>(cfg, env.sm_count); break;
    case KQ_BF16: e = configure_x<__nv_bfloat16>(cfg, env.sm_count); break;
    default: return cudaErrorInvalidValue;
  }
  if (e != cudaSuccess) return e;

  e = cudaMemcpyAsync(base + kStaticOpOff, &o, sizeof(o), cudaMemcpyHostToDevice, env.stream);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(base + kStaticBarOff, 0, 512, env.stream);  // barrier word and status word
  if (e != cudaSuccess) return e;
  PlanParams p = {};
  p.ops = reinterpret_cast<const PlanOpDev*>(base + kStaticOpOff);
  p.op_count = 1;
  p.m = m;
  p.partial = reinterpret_cast<float*>(base);
  p.counters = reinterpret_cast<unsigned int*>(base + kStaticCountersOff);
  p.grid_bar = reinterpret_cast<unsigned int*>(base + kStaticBarOff);
  p.error_flag = env.error_flag;
  p.status = reinterpret_cast<int*>(base + kStaticStatusOff);
  void* args[] = {&p};
  e = cudaLaunchCooperativeKernel(cfg.kernel, dim3(cfg.grid), dim3(kPlanWarps * 32), args, cfg.smem, env.stream);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyAsync(device_status, base + kStaticStatusOff, sizeof(int), cudaMemcpyDeviceToHost, env.stream);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(env.stream);
}

}  // namespace kq
