// qgemv_i4_tc — the small-batch int4 GEMV on Blackwell's tcgen05 tensor cores:
//   out[m, n] = x[m, k] . W[n, k]^T + bias   for 5 <= m <= 16 binary16 rows or 5 <= m <= 8
//   f32 / bf16 rows, W in the tiled int4 / group-32 layout (kq_common.cuh).
//
// Replaces the reference's small-M linear variants with in-kernel int4 dequant for the
// batched-decode / verify shapes (linear:v2:f32:reg*:wi4g32 —
// packages/runtime/src/kernels/gemm-geometry.ts:243-267; call site
// packages/runtime/src/runtime/recipe-builder.ts:1311-1392).
//
// The weights are the M side of the MMA (128 output rows per instruction), the activations
// the N side (16 columns), so one instruction does what 16 mma.sync would:
//
//   A (weights)  never touches shared memory as binary16.  A 512-byte chunk of the tiled
//                layout is already in mma-fragment order, and tcgen05.st.16x128b writes a
//                fragment-ordered register set into tensor memory exactly where
//                tcgen05.mma expects a K-major A tile (lane = output row, column = two
//                k-values).  A register holds two (u - 8) values: (word & mask) | 0x6400 is
//                the binary16 number 1024 + u (or 1024 + 16 u for the odd nibbles), and one
//                HSUB2 takes 1032 (1152) off, exactly.  The factor 16 of the odd nibbles is
//                taken out of the activations when they are staged.
//   B (x)        is converted once per launch by stage_x_tc_kernel into the K-major,
//                128-byte-swizzled image tcgen05.mma reads: 16 rows x 128 B per 64 k.  Every
//                activation row is pre-scaled by one power of two (pow2_prescale) and, for
//                f32 / bf16 input, split into a binary16 head (rows 0..7) and tail (rows
//                8..15) whose products are added in the epilogue.  A CTA copies the image
//                of its K slab into shared memory once.
//   D            one 128 x 16 f32 accumulator per scale group (two MMAs of K = 16), double
//                buffered in tensor memory; the warps read it back with tcgen05.ld and add
//                scale[row][group] * D to their f32 sums, the reference's per-group formula.
//
// A CTA is four teams of four warps; a team owns a quarter of the tensor memory columns,
// its own weight ring (cp.async.bulk + mbarrier) and its own sequence of 128-row tiles.
// All teams of a CTA work on the same K slab; with more than one slab the partial sums
// go to the context's scratch and tc_reduce_kernel adds them in slab order.
//
// Every wait is bounded; a wait that gives up sets the status word (reported by the next
// kq_sync as KQ_ERR_TIMEOUT) and a CTA-wide flag that lets all later waits return at once,
// so the kernel always reaches the tensor-memory deallocation.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

#include "kq_gemv_core.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kTeams = 4;
constexpr int kTcThreads = kTeams * 128 + kTeams * 32;  // the teams and one MMA-issuing warp for each
constexpr uint32_t kTcTileRows = 128;         // output rows per MMA
constexpr uint32_t kImageUnitBytes = 16 * 128;  // activations of 64 k: 16 rows x 128 B
constexpr uint32_t kTcWaitLimit = 1u << 22;
constexpr uint32_t kTcMaxSlots = 8;
constexpr size_t kTcSmemBudget = 227 * 1024;

struct TcParams {
  const uint8_t* w[kMaxMulti];
  const float* bias[kMaxMulti];
  float* out[kMaxMulti];
  uint32_t n[kMaxMulti];
  uint32_t row_begin[kMaxMulti];      // first row of the weight inside the concatenated output
  uint32_t tile_begin[kMaxMulti + 1];  // 128-row tiles, same order
  uint32_t count, m, k;
  uint32_t slabs, units_per_slab;  // K split; a unit is 64 k
  uint32_t slots, slot_units;      // ring slots per team; 64-k units of every row block in a slot
  uint32_t has_lo;                 // image rows 8..15 hold the tails of rows 0..7
  const uint8_t* image;            // [k / 64][16 x 128 B]
  const float* row_inv;            // [m]: 2^-e of every activation row
  float* partial;                  // [slabs][m][n_total] when slabs > 1
  uint32_t n_total;
  int* status;
};

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait; returns at once when another thread of the CTA already gave up.
__device__ __forceinline__ void tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  for (uint32_t spins = 0; spins < kTcWaitLimit; ++spins) {
    if (tc_mbar_try_wait(bar, parity)) return;
    if ((spins & 1023u) == 1023u && *abort_flag) return;
  }
  *abort_flag = 1;
  *reinterpret_cast<volatile int*>(status) = code;
}
__device__ __forceinline__ void team_sync(uint32_t team) {
  asm volatile("bar.sync %0, 128;" ::"r"(team + 1) : "memory");
}

// K-major, 128-byte swizzle: rows of 128 B, groups of 8 rows 1024 B apart, descriptor
// version 1, layout type 2 (the descriptor of kq_qgemm_i4.cu).
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(1) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) |
         (static_cast<uint64_t>(2) << 61);
}
// kind::f16: binary16 A and B (format 0), f32 accumulate, both K-major, M = 128, N = 16.
constexpr uint32_t kTcIdesc = (1u << 4) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(kTcIdesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Two nibbles of a word (selected by `mask`, 0x000F000F or 0x00F000F0) as two binary16
// values (u - 8) resp. 16 (u - 8): exact, two instructions.
__device__ __forceinline__ uint32_t nibbles_to_half2(uint32_t word, uint32_t mask, uint32_t bias_bits) {
  const uint32_t biased = (word & mask) | 0x64006400u;  // 1024 + u  (1024 + 16 u)
  const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&biased), *reinterpret_cast<const __half2*>(&bias_bits));
  return *reinterpret_cast<const uint32_t*>(&v);
}

// ---- the activation image ---------------------------------------------------------------
// One thread per (64-k unit, group of the unit, image row, octet): eight activations of one
// row become four 32-bit words of the image.  Inside a 32-k group the MMA's k index kk maps to
//   kk = 2t + h      -> element 8t + 2s + 4h          (s = which K-16 step of the group)
//   kk = 8 + 2t + h  -> element 8t + 2s + 1 + 4h, divided by 16
// which is the order the weight registers come out of a chunk (see nibbles_to_half2).
template <typename XT>
__global__ void __launch_bounds__(256)
stage_x_tc_kernel(const XT* __restrict__ x, uint32_t m, uint32_t k, const float* __restrict__ row_scale, uint8_t* image) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t q = item & 3u, row = (item >> 2) & 15u, jj = (item >> 6) & 1u, unit = item >> 7;
  if (unit >= k / 64) return;
  const bool is_lo = kHasLo && row >= 8;
  const uint32_t src_row = is_lo ? row - 8 : row;
  const bool live = src_row < m;
  uint32_t words[4] = {0, 0, 0, 0};  // {step 0 word q, step 0 word 4 + q, step 1 word q, step 1 word 4 + q}
  if (live) {
    float v[8];
    load_x8<XT>(x + static_cast<size_t>(src_row) * k + unit * 64 + jj * 32 + q * 8, v);
    const float scale = row_scale[src_row];
    __half h[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float staged = v[e] * ((e & 1) ? scale * 0.0625f : scale);
      h[e] = __float2half_rn(staged);
      if (is_lo) h[e] = __float2half_rn(staged - __half2float(h[e]));
    }
    words[0] = pack_half2(h[0], h[4]);
    words[1] = pack_half2(h[1], h[5]);
    words[2] = pack_half2(h[2], h[6]);
    words[3] = pack_half2(h[3], h[7]);
  }
  uint8_t* tile = image + static_cast<size_t>(unit) * kImageUnitBytes + row * 128;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t step = jj * 2 + (i >> 1), word = (i & 1) * 4 + q;
    const uint32_t chunk16 = step * 2 + (word >> 2);
    *reinterpret_cast<uint32_t*>(tile + ((chunk16 ^ (row & 7u)) * 16) + (word & 3u) * 4) = words[i];
  }
}

// out = bias + sum over slabs (ascending) of the partial sums.
__global__ void __launch_bounds__(256)
tc_reduce_kernel(const TcParams p) {
  const uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;  // row of the concatenated output
  if (col >= p.n_total) return;
  uint32_t wi = 0;
#pragma unroll
  for (int i = 1; i < kMaxMulti; ++i)
    if (i < static_cast<int>(p.count) && col >= p.row_begin[i]) wi = i;
  const uint32_t row = col - p.row_begin[wi];
  const float b = p.bias[wi][row];
  for (uint32_t mm = 0; mm < p.m; ++mm) {
    float total = 0.0f;
    for (uint32_t s = 0; s < p.slabs; ++s) total += p.partial[(static_cast<size_t>(s) * p.m + mm) * p.n_total + col];
    p.out[wi][static_cast<size_t>(mm) * p.n[wi] + row] = total + b;
  }
}

// ---- the matmul ---------------------------------------------------------------------------
// Shared memory (from a 1024-byte-aligned base):
//   [activation image of the slab: units_per_slab x 2 KB]
//   [weight rings: kTeams x slots x (8 row blocks x slot_units chunks)]
//   [mbarriers: image | full[team][slot] | done[team][2] | ready[team][2]] [tmem base, abort flag] [row_inv: 16 floats]
// Tensor memory, per team (128 columns): A buffers at +0 and +32 (64 k = 32 columns), D buffers
// at +64 and +96 (two groups x 16 columns).
template <bool kScaleF16>
__global__ void __launch_bounds__(kTcThreads, 1)
qgemv_i4_tc_kernel(const TcParams p) {
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;
  // a slot holds slot_units consecutive chunks of each of the tile's 8 row blocks: one copy per
  // row block, as long as the layout allows (the copy engine's rate is per copy, not per byte)
  const uint32_t kSlotBytes = 8u * p.slot_units * kCB;
  constexpr uint32_t kMask0 = 0x000F000Fu, kMask1 = 0x00F000F0u;
  constexpr uint32_t kBias1 = 0x64086408u, kBias16 = 0x64806480u;  // 1032, 1152 as binary16 pairs

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t tid = threadIdx.x, team = tid >> 7, tt = tid & 127u, tw = tt >> 5, lane = tid & 31u;
  const uint32_t image_bytes = p.units_per_slab * kImageUnitBytes;
  const uint32_t ring_base = base + image_bytes + team * p.slots * kSlotBytes;
  const uint32_t bars = base + image_bytes + kTeams * p.slots * kSlotBytes;
  const uint32_t bar_image = bars;
  const uint32_t bar_full = bars + 8 + team * (kTcMaxSlots * 8);
  const uint32_t bar_done_all = bars + 8 + kTeams * kTcMaxSlots * 8, bar_ready_all = bar_done_all + kTeams * 16;
  const uint32_t bar_done = bar_done_all + team * 16, bar_ready = bar_ready_all + team * 16;
  uint8_t* misc = smem + image_bytes + kTeams * p.slots * kSlotBytes + 8 + kTeams * kTcMaxSlots * 8 + kTeams * 32;
  uint32_t* tmem_word = reinterpret_cast<uint32_t*>(misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);
  float* inv_s = reinterpret_cast<float*>(misc + 16);

  if (tid == 0) {
    tc_mbar_init(bar_image, 1);
    for (uint32_t i = 0; i < kTeams; ++i) {
      for (uint32_t s = 0; s < kTcMaxSlots; ++s) tc_mbar_init(bars + 8 + (i * kTcMaxSlots + s) * 8, 1);
      tc_mbar_init(bar_done_all + i * 16, 1);       // one tcgen05.commit
      tc_mbar_init(bar_done_all + i * 16 + 8, 1);
      tc_mbar_init(bar_ready_all + i * 16, 4);      // one arrival per warp of the team
      tc_mbar_init(bar_ready_all + i * 16 + 8, 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (tid < 16) inv_s[tid] = tid < p.m ? p.row_inv[tid] : 0.0f;
  if (tid < 32) {
    const uint32_t slot_addr = static_cast<uint32_t>(__cvta_generic_to_shared(tmem_word));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const bool is_issuer = tid >= kTeams * 128;
  const uint32_t tmem = *tmem_word + (is_issuer ? 0u : team * 128u);

  // ---- which work is this team's ------------------------------------------------------
  const uint32_t slab = blockIdx.x % p.slabs, cta_in_slab = blockIdx.x / p.slabs;
  const uint32_t ctas_in_slab = (gridDim.x - slab + p.slabs - 1) / p.slabs;
  const uint32_t team_first = cta_in_slab * kTeams + team, team_stride = ctas_in_slab * kTeams;
  const uint32_t tiles = p.tile_begin[p.count];
  const uint32_t units = p.units_per_slab, chunks_per_row = p.k / kChunkK;

  // the slab's activation image: one thread starts the copies, every MMA issuer waits for them
  const bool cta_has_work = cta_in_slab * kTeams < tiles;
  if (tid == 0 && cta_has_work) {
    tc_mbar_expect_tx(bar_image, image_bytes);
    const uint8_t* src = p.image + static_cast<size_t>(slab) * image_bytes;
    for (uint32_t off = 0; off < image_bytes; off += 16384u)
      tc_bulk_g2s(base + off, src + off, min(16384u, image_bytes - off), bar_image);
  }

  // ---- the issuing warps: one thread per team feeds the tensor core -------------------------
  // Unit number q of a team uses A / D buffer q & 1; the team's warps arrive on ready[q & 1] once
  // their part of A is in tensor memory (and they are done with the D buffer's previous use).
  if (is_issuer) {
    const uint32_t t = (tid - kTeams * 128) >> 5;  // the team this warp issues for
    const uint32_t first = cta_in_slab * kTeams + t;
    if (lane == 0 && first < tiles) {
      const uint32_t total = ((tiles - first + team_stride - 1) / team_stride) * units;
      const uint32_t tm = *tmem_word + t * 128u;
      const uint64_t desc0 = tc_desc(base);
      tc_wait(bar_image, 0, abort_flag, p.status, 22);
      uint32_t unit = 0;
      for (uint32_t q = 0; q < total; ++q) {
        const uint32_t buf = q & 1u, parity = (q >> 1) & 1u;
        tc_wait(bar_ready_all + t * 16 + buf * 8, parity, abort_flag, p.status, 25);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t desc = desc0 + ((unit * kImageUnitBytes) >> 4);  // the start address field counts 16 bytes
#pragma unroll
        for (uint32_t step = 0; step < 4; ++step)
          tc_mma(tm + 64u + buf * 32u + (step >> 1) * 16u, tm + buf * 32u + step * 8u, desc + step * 2u, step & 1u);
        tc_commit(bar_done_all + t * 16 + buf * 8);
        unit = unit + 1 == units ? 0u : unit + 1;
      }
    }
  } else {
  // ---- the team's weight ring ---------------------------------------------------------------
  // Piece number q of the team (over all its tiles) goes to slot q % slots.
  auto locate = [&](uint32_t tile, uint32_t& wi, uint32_t& local_tile) {
    wi = 0;
#pragma unroll
    for (int i = 1; i < kMaxMulti; ++i)
      if (i < static_cast<int>(p.count) && tile >= p.tile_begin[i]) wi = i;
    local_tile = tile - p.tile_begin[wi];
  };
  const uint32_t slot_units = p.slot_units, pieces_per_tile = (units + slot_units - 1) / slot_units;
  uint32_t prod_q = 0;
  auto produce = [&]() {  // called by thread 32 of the team only
    const uint32_t job = prod_q / pieces_per_tile, piece = prod_q - job * pieces_per_tile;
    const uint32_t tile = team_first + job * team_stride;
    if (tile < tiles) {
      uint32_t wi, local_tile;
      locate(tile, wi, local_tile);
      const uint32_t rb0 = local_tile * 8u, nrb = min(8u, p.n[wi] / 16u - rb0);
      const uint32_t unit0 = piece * slot_units, nu = min(slot_units, units - unit0);
      const uint32_t slot = prod_q % p.slots;
      const uint32_t dst = ring_base + slot * kSlotBytes, bar = bar_full + slot * 8;
      tc_mbar_expect_tx(bar, nrb * nu * kCB);
      const uint8_t* src = p.w[wi] + (static_cast<size_t>(rb0) * chunks_per_row + slab * units + unit0) * kCB;
      for (uint32_t i = 0; i < nrb; ++i)
        tc_bulk_g2s(dst + i * slot_units * kCB, src + static_cast<size_t>(i) * chunks_per_row * kCB, nu * kCB, bar);
    }
    prod_q += 1;
  };
  if (tt == 32) {
    for (uint32_t s = 0; s < p.slots; ++s) produce();
  }

  const uint32_t row_in_tile = tw * 32u + lane;            // = this thread's tensor-memory lane
  const uint32_t my_rb = row_in_tile >> 4, my_rr = row_in_tile & 15u;
  const uint32_t scale_off = kChunkWeightBytes + ((my_rr & 7u) * 4u + (my_rr >> 3)) * kScaleBytes;  // group 0; +2 entries: group 1
  const uint32_t lane_field = (tw * 32u) << 16;

  uint32_t cons_q = 0;   // units consumed by the team (A / D buffer and its barrier's phase)
  uint32_t piece_q = 0;  // ring pieces consumed by the team
  for (uint32_t tile = team_first; tile < tiles; tile += team_stride) {
    uint32_t wi, local_tile;
    locate(tile, wi, local_tile);
    float acc[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[c] = 0.0f;
    float s_prev[2] = {0.0f, 0.0f};

    for (uint32_t unit = 0; unit <= units; ++unit) {
      const uint32_t buf = cons_q & 1u;
      float s_cur[2] = {0.0f, 0.0f};
      if (unit < units) {
        // (a) the unit's weights have landed
        const uint32_t in_piece = unit % slot_units;
        const uint32_t slot = piece_q % p.slots;
        if (in_piece == 0) tc_wait(bar_full + slot * 8, (piece_q / p.slots) & 1u, abort_flag, p.status, 21);
        const uint32_t slot_addr = ring_base + slot * kSlotBytes + in_piece * kCB;
        // (b) nibbles -> binary16 -> tensor memory: two row blocks per warp
#pragma unroll
        for (uint32_t half = 0; half < 2; ++half) {
          const uint32_t chunk = slot_addr + (tw * 2u + half) * slot_units * kCB;
          uint4 wv;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w) : "r"(chunk + lane * 16u));
          uint32_t r[16];
#pragma unroll
          for (int grp = 0; grp < 2; ++grp) {
            const uint32_t wa = grp ? wv.z : wv.x, wb = grp ? wv.w : wv.y;
            const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
            r[grp * 8 + 0] = nibbles_to_half2(wa, kMask0, kBias1);
            r[grp * 8 + 1] = nibbles_to_half2(wb, kMask0, kBias1);
            r[grp * 8 + 2] = nibbles_to_half2(wa, kMask1, kBias16);
            r[grp * 8 + 3] = nibbles_to_half2(wb, kMask1, kBias16);
            r[grp * 8 + 4] = nibbles_to_half2(wa8, kMask0, kBias1);
            r[grp * 8 + 5] = nibbles_to_half2(wb8, kMask0, kBias1);
            r[grp * 8 + 6] = nibbles_to_half2(wa8, kMask1, kBias16);
            r[grp * 8 + 7] = nibbles_to_half2(wb8, kMask1, kBias16);
          }
          const uint32_t taddr = tmem + lane_field + ((half * 16u) << 16) + buf * 32u;
          asm volatile(
              "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
              ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
              "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
              : "memory");
        }
        // this thread's two group scales of the unit (the slot is recycled before the drain)
        {
          const uint32_t sa = slot_addr + my_rb * slot_units * kCB + scale_off;
          if constexpr (kScaleF16) {
            unsigned short h0, h1;
            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h0) : "r"(sa));
            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h1) : "r"(sa + 2u * kScaleBytes));
            s_cur[0] = __half2float(__ushort_as_half(h0));
            s_cur[1] = __half2float(__ushort_as_half(h1));
          } else {
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s_cur[0]) : "r"(sa));
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s_cur[1]) : "r"(sa + 2u * kScaleBytes));
          }
        }
        // (c) this warp's part of A is in place (and it has drained the D buffer's previous use):
        // tell the issuing warp
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) tc_mbar_arrive(bar_ready + buf * 8);
        // after the last unit of a piece every warp of the team is done with the slot: refill it
        const bool piece_done = in_piece + 1 == slot_units || unit + 1 == units;
        if (piece_done) {
          team_sync(team);
          if (tt == 32) produce();
          piece_q += 1;
        }
        cons_q += 1;
      }
      // (d) the previous unit's accumulators: sums += scale * D, group by group
      if (unit > 0) {
        const uint32_t pq = (unit < units ? cons_q - 2 : cons_q - 1), pbuf = pq & 1u;
        tc_wait(bar_done + pbuf * 8, (pq >> 1) & 1u, abort_flag, p.status, 23);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t d[32];
        const uint32_t taddr = tmem + lane_field + 64u + pbuf * 32u;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]),
              "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]), "=r"(d[16]),
              "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]), "=r"(d[23]), "=r"(d[24]),
              "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          acc[c] = fmaf(s_prev[0], __uint_as_float(d[c]), acc[c]);
          acc[c] = fmaf(s_prev[1], __uint_as_float(d[16 + c]), acc[c]);
        }
      }
      s_prev[0] = s_cur[0];
      s_prev[1] = s_cur[1];
    }

    // ---- the tile's outputs: lane = output row --------------------------------------------
    const uint32_t row = local_tile * kTcTileRows + row_in_tile;
    if (row < p.n[wi]) {
      const float b = p.slabs == 1 ? p.bias[wi][row] : 0.0f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        if (static_cast<uint32_t>(c) >= p.m) break;
        float v = acc[c];
        if (p.has_lo && c < 8) v += acc[c + 8];
        v *= inv_s[c];
        if (p.slabs == 1)
          p.out[wi][static_cast<size_t>(c) * p.n[wi] + row] = v + b;
        else
          p.partial[(static_cast<size_t>(slab) * p.m + c) * p.n_total + p.row_begin[wi] + row] = v;
      }
    }
  }

  }  // teams
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*tmem_word), "r"(512u) : "memory");
  }
}

// ---- host side --------------------------------------------------------------------------
// How many K slabs: the CTAs of a slab share its 128-row tiles four teams at a time, so the
// time of a launch goes with (rounds of tiles per team) x (k per slab).  Among the splits whose
// activation image leaves room for a ring of at least three slots, the cheapest wins; ties go
// to fewer slabs (less partial-sum traffic).  A pure function of the shape.
struct TcShape {
  uint32_t slabs = 0, slots = 0, slot_units = 0;
  size_t smem = 0;
};

TcShape tc_shape(uint32_t tiles, uint32_t k, uint32_t m, uint32_t chunk_bytes, int sm_count) {
  TcShape best;
  uint64_t best_cost = ~0ull;
  const uint32_t units = k / kChunkK;
  const size_t fixed = 1024 + 8 + kTeams * kTcMaxSlots * 8 + kTeams * 32 + 16 + 64;
  for (uint32_t slabs = 1; slabs <= 16 && slabs <= units && slabs <= static_cast<uint32_t>(sm_count); slabs *= 2) {
    if (units % slabs != 0) break;
    const size_t image = static_cast<size_t>(units / slabs) * kImageUnitBytes;
    if (image + fixed >= kTcSmemBudget) continue;
    const size_t room = kTcSmemBudget - image - fixed;
    // the longest copies that still leave two slots; single-unit slots need three
    uint32_t slot_units = 0, slots = 0;
    for (uint32_t su : {4u, 2u, 1u}) {
      if (su > units / slabs && su != 1) continue;
      const size_t slot_bytes = static_cast<size_t>(kTeams) * 8 * su * chunk_bytes;
      const uint32_t fit = static_cast<uint32_t>(std::min<size_t>(kTcMaxSlots, room / slot_bytes));
      if (fit >= (su == 1 ? 3u : 2u)) {
        slot_units = su;
        slots = fit;
        break;
      }
    }
    if (slot_units == 0) continue;
    const uint32_t teams = (static_cast<uint32_t>(sm_count) / slabs) * kTeams;
    const uint64_t rounds = (tiles + teams - 1) / teams;
    // in units of 288 bytes moved: a (tile, unit) is 4608 B of weights; a (tile, slab) job of a
    // split launch writes and reads back 128 x m partial sums
    const uint64_t per_unit = slot_units == 4 ? 16 : slot_units == 2 ? 20 : 40;
    const uint64_t cost = rounds * ((units / slabs) * per_unit + (slabs > 1 ? (1024u * m) / 288u : 0u)) + (slabs > 1 ? 16 : 0);
    if (cost < best_cost) {
      best_cost = cost;
      best.slabs = slabs;
      best.slots = slots;
      best.slot_units = slot_units;
      best.smem = image + fixed + static_cast<size_t>(slots) * kTeams * 8 * slot_units * chunk_bytes;
    }
  }
  return best;
}

template <typename XT>
cudaError_t launch_tc_x(const LaunchEnv& env, TcParams& p, const void* x, bool f16s, int* launches) {
  constexpr bool kHasLo = !std::is_same<XT, __half>::value;
  const uint32_t chunk_bytes = kChunkWeightBytes + 32u * (f16s ? 2u : 4u);
  const uint32_t tiles = p.tile_begin[p.count];
  const TcShape shape = tc_shape(tiles, p.k, p.m, chunk_bytes, env.sm_count);
  if (shape.slabs == 0) return cudaErrorInvalidValue;
  p.slabs = shape.slabs;
  p.slots = shape.slots;
  p.slot_units = shape.slot_units;
  p.units_per_slab = p.k / kChunkK / shape.slabs;
  p.has_lo = kHasLo ? 1u : 0u;

  // scratch: [activation image][row scales: 16 scale + 16 inv][partial sums]
  const size_t image_bytes = static_cast<size_t>(p.k / kChunkK) * kImageUnitBytes;
  const size_t partial_bytes = shape.slabs > 1 ? static_cast<size_t>(shape.slabs) * p.m * p.n_total * sizeof(float) : 0;
  if (env.workspace == nullptr || image_bytes + 128 + partial_bytes > env.workspace_bytes) return cudaErrorMemoryAllocation;
  uint8_t* ws = static_cast<uint8_t*>(env.workspace);
  float* scale_ws = reinterpret_cast<float*>(ws + image_bytes);
  p.image = ws;
  p.row_inv = scale_ws + 16;
  p.partial = reinterpret_cast<float*>(ws + image_bytes + 128);
  p.status = env.status;

  row_scale_kernel<XT><<<p.m, 256, 0, env.stream>>>(static_cast<const XT*>(x), p.k, scale_ws, scale_ws + 16);
  const uint32_t items = (p.k / kChunkK) * 128u;
  stage_x_tc_kernel<XT><<<(items + 255) / 256, 256, 0, env.stream>>>(static_cast<const XT*>(x), p.m, p.k, scale_ws, ws);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  auto kernel = f16s ? qgemv_i4_tc_kernel<true> : qgemv_i4_tc_kernel<false>;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shape.smem));
  if (e != cudaSuccess) return e;
  const uint32_t quads = (tiles + kTeams - 1) / kTeams;  // CTAs a slab can keep busy
  const uint32_t per_slab = std::min<uint32_t>(quads, static_cast<uint32_t>(env.sm_count) / shape.slabs);
  kernel<<<per_slab * shape.slabs, kTcThreads, shape.smem, env.stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  int launched = 3;
  if (shape.slabs > 1) {
    tc_reduce_kernel<<<(p.n_total + 255) / 256, 256, 0, env.stream>>>(p);
    e = cudaGetLastError();
    launched += 1;
  }
  if (launches) *launches += launched;
  return e;
}

}  // namespace

bool qgemv_i4_tc_supports(int count, const LinearTarget* targets, int x_dtype, uint32_t m, int sm_count) {
  if (count < 1 || count > kMaxMulti) return false;
  if (x_dtype == KQ_F16 ? (m < 5 || m > 16) : (m < 5 || m > 8)) return false;
  const Weight& w0 = *targets[0].w;
  uint32_t tiles = 0;
  for (int i = 0; i < count; ++i) {
    const Weight& w = *targets[i].w;
    if (w.layout != kLayoutTiledI4 || w.k != w0.k || w.scale_dtype != w0.scale_dtype || w.n == 0) return false;
    tiles += (w.n + kTcTileRows - 1) / kTcTileRows;
  }
  const uint32_t chunk_bytes = kChunkWeightBytes + 32u * (w0.scale_dtype == KQ_F16 ? 2u : 4u);
  return tc_shape(tiles, w0.k, m, chunk_bytes, sm_count).slabs != 0;
}

cudaError_t launch_qgemv_i4_tc(const LaunchEnv& env, int count, const LinearTarget* targets, const void* x, int x_dtype,
                               uint32_t m, int* launches) {
  if (!qgemv_i4_tc_supports(count, targets, x_dtype, m, env.sm_count) || env.status == nullptr) return cudaErrorInvalidValue;
  TcParams p = {};
  p.count = static_cast<uint32_t>(count);
  p.m = m;
  p.k = targets[0].w->k;
  uint32_t tiles = 0, rows = 0;
  for (int i = 0; i < count; ++i) {
    const Weight& w = *targets[i].w;
    p.w[i] = static_cast<const uint8_t*>(w.data);
    p.bias[i] = targets[i].bias;
    p.out[i] = targets[i].out;
    p.n[i] = w.n;
    p.row_begin[i] = rows;
    p.tile_begin[i] = tiles;
    rows += w.n;
    tiles += (w.n + kTcTileRows - 1) / kTcTileRows;
  }
  for (int i = count; i <= kMaxMulti; ++i) p.tile_begin[i] = tiles;
  for (int i = count; i < kMaxMulti; ++i) p.row_begin[i] = rows;
  p.n_total = rows;
  const bool f16s = targets[0].w->scale_dtype == KQ_F16;
  switch (x_dtype) {
    case KQ_F32: return launch_tc_x<float>(env, p, x, f16s, launches);
    case KQ_F16: return launch_tc_x<__half>(env, p, x, f16s, launches);
    case KQ_BF16: return launch_tc_x<__nv_bfloat16>(env, p, x, f16s, launches);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace kq
