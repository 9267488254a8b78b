// qgemm_i4 — the prefill kernels of libkq: out[m, n] = x[m, k] . W[n, k]^T + bias for large m,
// bf16 activations, W in the tiled int4 / group-32 or the tiled int8 layout (kq_common.cuh).
//
// Replaces the reference's large-M linear variants with in-kernel dequant
// (linear:v2:f32:reg64x32r4x4w8:wi4g32 and reg128x128r8x8w16 —
// packages/runtime/src/kernels/gemm-geometry.ts:243-267, kernel text
// packages/runtime/tests/fixtures/wgsl/linear_wi4_v4.wgsl): the same "dequantise a weight
// tile into shared memory, then contract" structure, on Blackwell's tensor cores.
//
// One body, two forms.
//
// Single CTA (at most 256 activation rows):
//   CTA tile 256 (m) x 256 (n), k-step 64, three shared-memory stages of 64 KB.
//   warps 0-15 producers.  Per k-step they copy the 256 x 64 bf16 activation tile (cp.async,
//              straight into the swizzled tile) and dequantise the 256 x 64 weight tile (16-row
//              blocks of the tiled layout, read with 128-bit loads one k-step ahead) into the
//              canonical K-major 128-byte-swizzled layout that tcgen05.mma reads.  A dequantised
//              element is RNE_bf16(fround((u - 8) * s)) or RNE_bf16(fround(q * s)): the
//              reference's single-rounding f32 value (kq::dequant_i4 / dequant_i8, computed
//              with an exact integer-to-float trick instead of a conversion), rounded once
//              more to the tensor core's input type.  After the main loop they drain the
//              accumulators.
//   warp 16    one elected thread issues tcgen05.mma (M 128 x N 256 x K 16, bf16 in, f32
//              accumulate) — two per k16 slice, one per 128-row half of the tile, sharing
//              the weight operand — and commits each stage back to the producers.
//   TMEM       512 columns: two 128 x 256 f32 accumulators.
//
// CTA pair (more than 256 rows): a cluster of two CTAs = two consecutive 256-row tiles of the
//   same 256 output channels runs ONE tcgen05.mma.cta_group::2 stream (M 256 = 128 rows of each
//   CTA, N 256).  Each CTA keeps its own activation tile and accumulators and dequantises only
//   HALF of the weight tile; the tensor cores read the other half from the peer's shared
//   memory.  Stages are 48 KB, four of them.  The producers work as two groups of eight warps
//   that fill alternate k-steps, and a group starts the activation copy of its next k-step as
//   soon as it has handed the current stage over: the waits, fences and arrivals that end a
//   step (each costs a memory round trip or more while loads are in flight) overlap the other
//   group's arithmetic.  The CTA of cluster rank 0 issues the MMAs; the peer's producers
//   arrive on its "full" barriers, and it commits each stage to both CTAs' "empty" barriers.
//   Shapes whose last wave of tiles would idle the machine are streamed: one persistent pair
//   per SM pair takes a contiguous run of (tile, k-step) units, and a tile cut between two
//   pairs is summed through scratch by the pair that holds its first k-step.
//
// Parity contract (there is no bf16-compute variant in the reference): the result equals
// the reference's math (f64-accumulate oracle) applied to the bf16 activations and to the
// bf16-rounded dequantised weights, within atol 1e-5 + rtol 1e-3.
//
// Every mbarrier wait and every flag wait is bounded; a wait that gives up sets a status word
// and a CTA-wide abort flag that makes all later waits return at once, so the kernel always
// reaches the TMEM deallocation and exits.
#include <cuda.h>
#include <cuda_bf16.h>

#include <type_traits>

#include "kq_common.cuh"
#include "kq_gemm_stream.h"
#include "kq_umma.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

using namespace umma;

constexpr int kBM = 256, kBN = 256, kBK = 64, kStagesG = 3;
#ifndef KQ_GEMM_PRODUCER_WARPS
#define KQ_GEMM_PRODUCER_WARPS 16
#endif
constexpr int kProducerWarps = KQ_GEMM_PRODUCER_WARPS;  // 8 or 16
#ifndef KQ_GEMM_PAIR_STAGES
#define KQ_GEMM_PAIR_STAGES 4  // 2 .. 4 (four stages of 48 KB fill the shared memory)
#endif
constexpr int kGemmThreads = kProducerWarps * 32 + 32;
constexpr uint32_t kATileBytes = kBM * kBK * 2;  // 32 KB
constexpr uint32_t kBTileBytes = kBN * kBK * 2;  // 32 KB
constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;
constexpr uint32_t kTmemCols = 512;

struct GemmParams {
  const uint8_t* w;  // tiled int4 weight (scales inside the chunks) or tiled int8 weight
  const void* scale;  // int8 only: the per-output-channel scales, [n]
  const __nv_bfloat16* x;
  const float* bias;
  float* out;
  uint32_t m, n, k;
  int* status;
  // K split over blockIdx.z: each slice accumulates ksteps_per_split k-steps and, when there is
  // more than one slice, leaves its partial sums (no bias) in partial[z][m][n].
  uint32_t ksteps_per_split, splits;
  float* partial;
  // Pair form, stream_pairs != 0: the launch is stream_pairs clusters and the pair tiles x k-steps
  // are dealt to them as one contiguous run each (pair tile t = column tile t / m_pairs, row
  // pair t % m_pairs).  A pair that starts inside a tile leaves that piece's sums in its slot
  // (slots[pair][cta][256][256]) and raises flags[2 * pair + cta]; the pair that holds the tile's
  // first k-step adds the slots of the pairs after it, in order, before it stores.
  uint32_t stream_pairs, pair_tiles, m_pairs;
  float* slots;
  unsigned int* flags;
};

// Four bytes q + 128 of one weight row -> four bf16 values RNE_bf16(fround(q * s)).  A byte
// placed under the exponent of 2^23 reads as the float 2^23 + byte exactly; subtracting
// 2^23 + 128 leaves q exactly, so the multiply's rounding is the reference's only one
// (kq::dequant_i8's rule).
__device__ __forceinline__ uint2 dequant4_i8_bf16(uint32_t word, float s) {
  const float v0 = (__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7650u)) - 8388736.0f) * s;
  const float v1 = (__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7651u)) - 8388736.0f) * s;
  const float v2 = (__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7652u)) - 8388736.0f) * s;
  const float v3 = (__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7653u)) - 8388736.0f) * s;
  uint2 out;
  __nv_bfloat162 q;
  q = __floats2bfloat162_rn(v0, v1); out.x = *reinterpret_cast<uint32_t*>(&q);
  q = __floats2bfloat162_rn(v2, v3); out.y = *reinterpret_cast<uint32_t*>(&q);
  return out;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint2 v) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(v.x), "r"(v.y) : "memory");
}

// kPair: the two CTAs of a cluster (consecutive blockIdx.x = consecutive 256-row tiles of m, the
// same 256 output channels) run ONE tcgen05.mma.cta_group::2 stream: each CTA keeps its own
// activation tile and accumulators, and dequantises only half of the weight tile (128
// channels) — the tensor core reads the other half from the peer's shared memory.  The MMAs are
// issued by the CTA of cluster rank 0; the peer's producers arrive on that CTA's "full"
// barriers, and each commit is sent to both CTAs' "empty" barriers.
template <bool kInt8, bool kScaleF16, bool kPair, int kGroups>
__device__ __forceinline__ void qgemm_body(const GemmParams& p, const CUtensorMap* x_map) {
  // Pair form, int4 weights: a stage's activation tile is ONE tensor-map copy (TMA, 128-byte
  // swizzle, rows past m filled with zeros) started by one thread of the filling group; both
  // CTAs' copies report their bytes straight to the issuing CTA's "full" barrier.  The other
  // forms copy 16-byte pieces with cp.async (with int8 weights the tensor-map copy measured
  // 5-6 % slower, twice; with int4 weights 1-6 % faster).
  constexpr bool kTmaA = kPair && !kInt8;
  static_assert(!kPair || (kProducerWarps == 16 && kGroups == 2), "the pair form: two groups of 8 warps");
  // The producer warps work in kGroups groups, group j filling the stages of k-steps j, j + kGroups, ...:
  // while one group sits in its barrier wait, fences and arrival, the other computes.
  constexpr int kGW = kProducerWarps / kGroups;           // warps per group
  constexpr int kChunksPerWarp = (kPair ? 8 : 16) / kGW;  // 16-row weight blocks per warp and k-step
  constexpr int kAPiecesPerThread = 2048 / (kGW * 32);
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;
  constexpr int kStagesG = kPair ? KQ_GEMM_PAIR_STAGES : kq::kStagesG;  // a pair's stage is 48 KB instead of 64
  constexpr uint32_t kStageBytes = kATileBytes + (kPair ? kBTileBytes / 2 : kBTileBytes);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t raw_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
  const uint32_t tiles = (raw_base + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t bars = tiles + kStagesG * kStageBytes;  // full[stages], empty[stages], accum
  const uint32_t tmem_slot = bars + 96;
  uint8_t* generic_base = smem_raw + (tiles - raw_base);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(generic_base + kStagesG * kStageBytes + 104);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + kStagesG * kStageBytes + 96);
  const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;

  const uint32_t chunks_per_row = p.k / kChunkK, ksteps_all = p.k / kBK;
  // What this CTA computes, as a list of fragments (tile, k range).  Without streaming there is one:
  // the tile and K slice the block index names.  With streaming the pair's run of units is cut
  // at the tile boundaries.
  const bool streaming = kPair && p.stream_pairs != 0;
  const uint32_t pair_index = blockIdx.x >> 1;
  const uint64_t units = static_cast<uint64_t>(p.pair_tiles) * ksteps_all;
  uint32_t unit_begin = 0, unit_end = 0, frag_count = 1;
  if (streaming) {
    unit_begin = stream::run_begin(pair_index, units, p.stream_pairs);
    unit_end = stream::run_begin(pair_index + 1, units, p.stream_pairs);
    frag_count = stream::fragment_count(unit_begin, unit_end, ksteps_all);
  }
  using stream::kFinal; using stream::kSlice; using stream::kPiece; using stream::kOwner;
  // the current fragment: tile origin, first k-step, k-steps, what happens to the sums, the unit
  // after the tile's last, and how many k-steps this CTA ran before (stages and phases count on)
  uint32_t n0 = 0, m0 = 0, ks_begin = 0, ksteps = 0, kind = kFinal, tile_end_unit = 0, it_base = 0;
  auto select_fragment = [&](uint32_t f) {
    if (streaming) {
      const stream::Fragment fr = stream::fragment(unit_begin, unit_end, ksteps_all, f);
      ks_begin = fr.ks_begin;
      ksteps = fr.ksteps;
      tile_end_unit = fr.tile_end_unit;
      kind = fr.kind;
      n0 = (fr.tile / p.m_pairs) * kBN;
      m0 = ((fr.tile % p.m_pairs) * 2u + cta_rank) * kBM;
    } else {
      // a pair lies along x (the hardware pairs CTAs of consecutive cluster rank): there x walks m
      n0 = (kPair ? blockIdx.y : blockIdx.x) * kBN;
      m0 = (kPair ? blockIdx.x : blockIdx.y) * kBM;
      ks_begin = blockIdx.z * p.ksteps_per_split;
      ksteps = min(ks_begin + p.ksteps_per_split, ksteps_all) - ks_begin;
      kind = p.splits == 1 ? kFinal : kSlice;
    }
  };
  const uint32_t tmem_free = bars + 72;  // pair form: both CTAs have drained the accumulators of a fragment

  if (warp == kProducerWarps) {
    if (lane == 0) {
      for (int s = 0; s < kStagesG; ++s) {
        mbar_init(bars + s * 8, (kPair ? 2 : 1) * kGW * 32 + (kTmaA ? 1 : 0));  // full: every thread of the filling group (of both CTAs) arrives; + the tensor copies' bytes
        mbar_init(bars + (kStagesG + s) * 8, 1);       // empty: one tcgen05.commit
      }
      mbar_init(bars + 2 * kStagesG * 8, 1);           // accumulators complete
      mbar_init(tmem_free, kPair ? 2 : 1);
      *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if constexpr (kPair) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if constexpr (kPair) cluster_sync_all();  // the peer's barriers are initialised before anyone arrives on them
  else __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp < kProducerWarps) {
    // ---------------- producers ----------------
    const uint32_t grp = warp / kGW, wg = warp % kGW;  // group, warp within it
    const uint32_t tid = threadIdx.x % (kGW * 32u);    // thread within the group
    const uint32_t g = lane >> 2, t = lane & 3u;
    for (uint32_t f = 0; f < frag_count; ++f) {
    select_fragment(f);
    // group j fills the stages of the k-steps whose running count is j modulo the group count
    const uint32_t ks_first = (grp + kGroups - it_base % kGroups) % kGroups;
    // The lane's two weight chunks (and their scales) of a k-step, fetched one k-step ahead.
    uint4 wq_next[kChunksPerWarp];
    typename std::conditional<kScaleF16, uint2, uint4>::type sc_next[kChunksPerWarp];
    // Addresses that only advance by a constant per k-step are kept in registers: the lane's
    // word of each of its chunks (next k-step: + one chunk) ...
    const uint8_t* chunk_ptr[kChunksPerWarp];
    bool chunk_live[kChunksPerWarp];
#pragma unroll
    for (int cc = 0; cc < kChunksPerWarp; ++cc) {
      // first output channel of the row block; in a pair two warps share a block of this CTA's 128 channels
      const uint32_t row0 = n0 + (kPair ? cta_rank * 128u : 0u) + (wg * kChunksPerWarp + cc) * 16u;
      chunk_live[cc] = row0 < p.n;
      chunk_ptr[cc] = p.w + (static_cast<size_t>(row0 >> 4) * chunks_per_row + ks_begin + ks_first) * kCB + lane * 16;
    }
    const uint32_t scale_off = kChunkWeightBytes - lane * 16 + g * (kScaleF16 ? 8u : 16u);
    // int8: a 16-row block's k-step is two adjacent 512-byte chunks (32 k each), one 16-byte
    // read per lane and chunk; the two rows' scales do not change along k.
    uint4 w8_next[kChunksPerWarp][2];
    float s8[kChunksPerWarp][2];
    if constexpr (kInt8) {
#pragma unroll
      for (int cc = 0; cc < kChunksPerWarp; ++cc) {
        const uint32_t row0 = n0 + (kPair ? cta_rank * 128u : 0u) + (wg * kChunksPerWarp + cc) * 16u;
        chunk_ptr[cc] = p.w + (static_cast<size_t>(row0 >> 4) * (p.k / kChunkK8) + (ks_begin + ks_first) * 2u) * 512u + lane * 16;
        s8[cc][0] = chunk_live[cc] ? load_scale<kScaleF16>(p.scale, row0 + g) : 0.0f;
        s8[cc][1] = chunk_live[cc] ? load_scale<kScaleF16>(p.scale, row0 + g + 8u) : 0.0f;
      }
    }
    auto fetch_weights = [&](uint32_t ks) {
      if constexpr (kInt8) {
#pragma unroll
        for (int cc = 0; cc < kChunksPerWarp; ++cc) {
          w8_next[cc][0] = w8_next[cc][1] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);  // q = 0
          if (chunk_live[cc] && ks < ksteps) {
            w8_next[cc][0] = *reinterpret_cast<const uint4*>(chunk_ptr[cc]);
            w8_next[cc][1] = *reinterpret_cast<const uint4*>(chunk_ptr[cc] + 512);
            chunk_ptr[cc] += 1024 * kGroups;
          }
        }
        return;
      }
#pragma unroll
      for (int cc = 0; cc < kChunksPerWarp; ++cc) {
        wq_next[cc] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);  // u = 8 -> value 0
        if constexpr (kScaleF16) sc_next[cc] = make_uint2(0, 0);
        else sc_next[cc] = make_uint4(0, 0, 0, 0);
        if (chunk_live[cc] && ks < ksteps) {
          wq_next[cc] = *reinterpret_cast<const uint4*>(chunk_ptr[cc]);
          if constexpr (kScaleF16) sc_next[cc] = *reinterpret_cast<const uint2*>(chunk_ptr[cc] + scale_off);
          else sc_next[cc] = *reinterpret_cast<const uint4*>(chunk_ptr[cc] + scale_off);
          chunk_ptr[cc] += kCB * kGroups;
        }
      }
    };
    // ... and the source and the swizzled destination offset of the thread's activation pieces
    // (next k-step: + 64 elements; the stage base is added per step)
    const __nv_bfloat16* a_src[kAPiecesPerThread];
    uint32_t a_dst[kAPiecesPerThread], a_bytes[kAPiecesPerThread];
#pragma unroll
    for (int i = 0; i < (kTmaA ? 0 : kAPiecesPerThread); ++i) {
      const uint32_t piece = tid + i * (kGW * 32u);
      const uint32_t r = piece >> 3, c = piece & 7u;
      const bool in_range = m0 + r < p.m;
      a_src[i] = p.x + static_cast<size_t>(in_range ? m0 + r : 0) * p.k + (ks_begin + ks_first) * kBK + c * 8;
      a_dst[i] = swz(r, c);
      a_bytes[i] = in_range ? 16u : 0u;
    }
    // activations: 256 rows x 8 pieces of 16 B, copied asynchronously straight into the swizzled
    // tile of the k-step's stage (rows past m are zero-filled), once that stage is free
    auto copy_activations = [&](uint32_t ks) {
      if (ks < ksteps) {
        const uint32_t it = it_base + ks, s = it % kStagesG, phase = (it / kStagesG) & 1u;
        wait_bounded(bars + (kStagesG + s) * 8, phase ^ 1u, abort_flag, p.status, 1);
        const uint32_t a_tile = tiles + s * kStageBytes;
        if constexpr (kTmaA) {
          if (tid == 0) {
            // Both CTAs' copies report their bytes to the issuing CTA's "full" barrier (the
            // cta_group::2 form of the copy may signal a barrier of the peer CTA), which that CTA
            // arms for the two tiles: no thread has to wait for the tile and vouch for it.
            const uint32_t full_bar = map_to_cta(bars + s * 8, 0);
            if (cta_rank == 0)
              asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bars + s * 8), "r"(2u * kATileBytes) : "memory");
            asm volatile(
                "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                ::"r"(a_tile), "l"(x_map), "r"((ks_begin + ks) * kBK), "r"(m0), "r"(full_bar)
                : "memory");
          }
        } else {
#pragma unroll
          for (int i = 0; i < kAPiecesPerThread; ++i) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a_tile + a_dst[i]), "l"(a_src[i]), "r"(a_bytes[i])
                         : "memory");
            a_src[i] += kBK * kGroups;
          }
        }
      }
      if constexpr (!kTmaA) asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // With groups, a group's copy for its NEXT k-step starts as soon as the current stage is
    // handed over: its latency then overlaps the whole next dequant instead of ending the step.
    constexpr bool kCopyAhead = kGroups > 1;
    fetch_weights(ks_first);
    if constexpr (kCopyAhead) copy_activations(ks_first);
    for (uint32_t ks = ks_first; ks < ksteps; ks += kGroups) {
      const uint32_t s = (it_base + ks) % kStagesG;
      if constexpr (!kCopyAhead) copy_activations(ks);  // the copy flies while we dequantise
      const uint32_t a_tile = tiles + s * kStageBytes, b_tile = a_tile + kATileBytes;
      if constexpr (kInt8) {
        uint4 w8[kChunksPerWarp][2];
#pragma unroll
        for (int cc = 0; cc < kChunksPerWarp; ++cc) { w8[cc][0] = w8_next[cc][0]; w8[cc][1] = w8_next[cc][1]; }
        fetch_weights(ks + kGroups);
#pragma unroll
        for (int cc = 0; cc < kChunksPerWarp; ++cc) {
          // chunk j, words x | y | z | w = row g k 4t.. | row g+8 same k | row g k 16+4t.. | row g+8:
          // four weights = 8 bytes = half (t & 1) of 16-byte piece 4j + 2h + (t >> 1) of the tile
          // row.  The 16 lanes of a shared-memory phase (four values of g) must hit 8 different
          // swizzled pieces: the order in which a lane walks its four (j, h) pairs is XORed with
          // a value that differs where the rows' swizzle term (g >> 1) does not.
          const uint32_t r_a = (wg * kChunksPerWarp + cc) * 16u + g, r_b = r_a + 8u;
          const bool odd = (g & 1u) != 0;
          const uint32_t sub = (t >> 1), byte = (t & 1u) * 8u;
          uint2 da[4], db[4];  // index 2j + h
          da[0] = dequant4_i8_bf16(w8[cc][0].x, s8[cc][0]); db[0] = dequant4_i8_bf16(w8[cc][0].y, s8[cc][1]);
          da[1] = dequant4_i8_bf16(w8[cc][0].z, s8[cc][0]); db[1] = dequant4_i8_bf16(w8[cc][0].w, s8[cc][1]);
          da[2] = dequant4_i8_bf16(w8[cc][1].x, s8[cc][0]); db[2] = dequant4_i8_bf16(w8[cc][1].y, s8[cc][1]);
          da[3] = dequant4_i8_bf16(w8[cc][1].z, s8[cc][0]); db[3] = dequant4_i8_bf16(w8[cc][1].w, s8[cc][1]);
#pragma unroll
          for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t o = odd ? (i ^ 2u) : i;  // the (j, h) pair of this store
            const uint2 va = odd ? da[i ^ 2u] : da[i], vb = odd ? db[i ^ 2u] : db[i];
            sts64(b_tile + swz(r_a, o * 2u + sub) + byte, va);
            sts64(b_tile + swz(r_b, o * 2u + sub) + byte, vb);
          }
        }
      } else {
      // weights: this k-step's chunks are already in registers; fetch the next k-step's
      uint4 wq[kChunksPerWarp];
      float sc[kChunksPerWarp][4];
#pragma unroll
      for (int cc = 0; cc < kChunksPerWarp; ++cc) {
        wq[cc] = wq_next[cc];
        if constexpr (kScaleF16) {
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&sc_next[cc].x));
          const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&sc_next[cc].y));
          sc[cc][0] = a.x; sc[cc][1] = a.y; sc[cc][2] = b.x; sc[cc][3] = b.y;
        } else {
          sc[cc][0] = __uint_as_float(sc_next[cc].x); sc[cc][1] = __uint_as_float(sc_next[cc].y);
          sc[cc][2] = __uint_as_float(sc_next[cc].z); sc[cc][3] = __uint_as_float(sc_next[cc].w);
        }
      }
      fetch_weights(ks + kGroups);
#pragma unroll
      for (int cc = 0; cc < kChunksPerWarp; ++cc) {
        // words: row g grp 0 | row g+8 grp 0 | row g grp 1 | row g+8 grp 1; the lane's 8
        // nibbles of a group are k = 8t .. 8t+7 of that group = 16-byte piece t (group 0)
        // or 4 + t (group 1) of the 128-byte tile row.  Odd g stores group 1 first: the 8
        // lanes of a shared-memory phase (two values of g, four of t) then hit 8 different
        // 16-byte columns of the swizzled rows.
        const uint32_t r_a = (wg * kChunksPerWarp + cc) * 16u + g, r_b = r_a + 8u;
        const uint4 a0 = dequant8_bf16(wq[cc].x, sc[cc][0]), a1 = dequant8_bf16(wq[cc].z, sc[cc][2]);
        const uint4 b0 = dequant8_bf16(wq[cc].y, sc[cc][1]), b1 = dequant8_bf16(wq[cc].w, sc[cc][3]);
        const bool odd = (g & 1u) != 0;
        sts128(b_tile + swz(r_a, odd ? 4u + t : t), odd ? a1 : a0);
        sts128(b_tile + swz(r_a, odd ? t : 4u + t), odd ? a0 : a1);
        sts128(b_tile + swz(r_b, odd ? 4u + t : t), odd ? b1 : b0);
        sts128(b_tile + swz(r_b, odd ? t : 4u + t), odd ? b0 : b1);
      }
      }
      if constexpr (!kTmaA) asm volatile("cp.async.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
      if (kPair && cta_rank != 0) mbar_arrive_cluster(map_to_cta(bars + s * 8, 0));  // the issuing CTA's barrier
      else mbar_arrive(bars + s * 8);
      if constexpr (kCopyAhead) copy_activations(ks + kGroups);
    }
    // ---------------- epilogue: accumulators -> out ----------------
    it_base += ksteps;
    wait_bounded(bars + 2 * kStagesG * 8, f & 1u, abort_flag, p.status, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // kOwner: the pairs after this one that hold pieces of the tile; their flags must be up
    uint32_t partners = 0;
    if (kind == kOwner) {
      partners = stream::partners(pair_index, tile_end_unit, units, p.stream_pairs);
      if (lane == 0) {
        for (uint32_t q = 1; q <= partners; ++q) {
          const unsigned int* flag = p.flags + (pair_index + q) * 2u + cta_rank;
          uint32_t spins = 0, up = 0;
          while (up == 0 && spins < kWaitLimit && !*abort_flag) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(up) : "l"(flag) : "memory");
            ++spins;
          }
          if (up == 0 && !*abort_flag) {
            *abort_flag = 1;
            *reinterpret_cast<volatile int*>(p.status) = 6;
          }
        }
      }
      __syncwarp();
    }
    const size_t slot_floats = static_cast<size_t>(kBM) * kBN;
    // a warp may only touch the TMEM lane quarter warp % 4; the warps sharing a quarter split
    // the two accumulators (rows 0-127 / 128-255) and, with 16 producers, the column halves
    const uint32_t quarter = warp & 3u, group = warp >> 2;
    const uint32_t half = group & 1u;
    constexpr uint32_t kColBatches = (kBN / 32) / (kProducerWarps / 8);
    const uint32_t cb0 = (group >> 1) * kColBatches;
    const uint32_t row = m0 + half * 128u + quarter * 32u + lane;
#pragma unroll 1
    for (uint32_t cb = cb0; cb < cb0 + kColBatches; ++cb) {
      uint32_t v[32];
      const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + half * kBN + cb * 32u;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
          "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
            "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
            "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
            "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      // A lane holds 32 consecutive outputs of ONE row: stored like that, a warp's store touches
      // 32 different lines, 16 bytes each.  The batch goes through shared memory (the stage
      // buffers are free: the last MMA has completed) and leaves transposed — one coalesced
      // 128-byte store per row (wider stores, four rows each, measured slightly slower).  Row
      // stride 36 floats: both the 16-byte writes and the 4-byte reads are bank-conflict free.
      const uint32_t col0 = n0 + cb * 32u;
      float* scratch = reinterpret_cast<float*>(generic_base) + warp * (32u * 36u);
      __syncwarp();  // the previous batch has been read
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(scratch + lane * 36u + j) =
            make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      __syncwarp();
      const bool final_sum = kind == kFinal;
      const uint32_t col = col0 + lane;
      if (kind == kPiece) {
        // a piece of a tile: the whole 256 x 256 block of sums, no bias, into this CTA's slot
        float* dst = p.slots + (pair_index * 2u + cta_rank) * slot_floats + (half * 128u + quarter * 32u) * kBN + cb * 32u + lane;
        for (uint32_t rr = 0; rr < 32u; ++rr) dst[rr * kBN] = scratch[rr * 36u + lane];
      } else if (kind == kOwner) {
        if (col < p.n) {
          const float b = p.bias[col];
          const uint32_t row_first = row - lane;
          const uint32_t rows_here = row_first < p.m ? min(32u, p.m - row_first) : 0u;
          const float* piece = p.slots + ((pair_index + 1u) * 2u + cta_rank) * slot_floats + (half * 128u + quarter * 32u) * kBN + cb * 32u + lane;
          // all of a piece's 32 loads are in flight together (one after the other, each row would
          // cost a trip to memory); pieces are added in pair order
          float sums[32];
#pragma unroll
          for (uint32_t rr = 0; rr < 32u; ++rr) sums[rr] = scratch[rr * 36u + lane];
          for (uint32_t q = 0; q < partners; ++q) {
            float piece_rows[32];
#pragma unroll
            for (uint32_t rr = 0; rr < 32u; ++rr) piece_rows[rr] = __ldcg(piece + q * 2u * slot_floats + rr * kBN);
#pragma unroll
            for (uint32_t rr = 0; rr < 32u; ++rr) sums[rr] += piece_rows[rr];
          }
#pragma unroll
          for (uint32_t rr = 0; rr < 32u; ++rr)
            if (rr < rows_here) p.out[static_cast<size_t>(row_first + rr) * p.n + col] = sums[rr] + b;
        }
      } else if (col < p.n) {
        const float b = final_sum ? p.bias[col] : 0.0f;
        const uint32_t row_first = row - lane;  // first row of this warp's 32
        float* dst = (final_sum ? p.out : p.partial + static_cast<size_t>(blockIdx.z) * p.m * p.n) + col;
        const uint32_t rows_here = row_first < p.m ? min(32u, p.m - row_first) : 0u;
        for (uint32_t rr = 0; rr < rows_here; ++rr)
          dst[static_cast<size_t>(row_first + rr) * p.n] = scratch[rr * 36u + lane] + b;
      }
    }
    if (streaming) {
      // Every producer warp has drained its part of the accumulators and left its scratch (the
      // stage buffers) before the next fragment starts; then one thread publishes the piece,
      // lowers the flags it consumed, and tells the issuing CTA that TMEM may be overwritten.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // scratch reads and writes before the next tile copies land there
      asm volatile("bar.sync 1, %0;" ::"r"(kProducerWarps * 32) : "memory");
      if (threadIdx.x == 0) {
        if (kind == kPiece) {
          __threadfence();
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.flags + pair_index * 2u + cta_rank), "r"(1u) : "memory");
        } else if (kind == kOwner) {
          for (uint32_t q = 1; q <= partners; ++q) p.flags[(pair_index + q) * 2u + cta_rank] = 0u;
        }
        if (f + 1 < frag_count) mbar_arrive_cluster(map_to_cta(tmem_free, 0));
      }
    }
    }  // fragments
  } else if (cta_rank == 0) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t kIdesc = umma_idesc(kPair ? 256 : 128, kBN);
    for (uint32_t f = 0; f < frag_count; ++f) {
    select_fragment(f);
    if (f != 0) {  // both CTAs have read the previous fragment's sums out of TMEM
      wait_bounded_cluster(tmem_free, (f - 1u) & 1u, abort_flag, p.status, 7);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    for (uint32_t ks = 0; ks < ksteps; ++ks) {
      const uint32_t it = it_base + ks, s = it % kStagesG, phase = (it / kStagesG) & 1u;
      const bool ok = kPair ? wait_bounded_cluster(bars + s * 8, phase, abort_flag, p.status, 2)
                            : wait_bounded(bars + s * 8, phase, abort_flag, p.status, 2);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint32_t a_tile = tiles + s * kStageBytes, b_tile = a_tile + kATileBytes;
        if (ok) {
#pragma unroll
          for (uint32_t kk = 0; kk < kBK / 16; ++kk) {
            const uint64_t db = umma_desc(b_tile + kk * 32u);
            const uint32_t acc = (ks | kk) != 0 ? 1u : 0u;
            if constexpr (kPair) {
              umma_bf16_pair(tmem_base, umma_desc(a_tile + kk * 32u), db, kIdesc, acc);
              umma_bf16_pair(tmem_base + kBN, umma_desc(a_tile + 128u * 128u + kk * 32u), db, kIdesc, acc);
            } else {
              umma_bf16(tmem_base, umma_desc(a_tile + kk * 32u), db, kIdesc, acc);
              umma_bf16(tmem_base + kBN, umma_desc(a_tile + 128u * 128u + kk * 32u), db, kIdesc, acc);
            }
          }
        }
        // the stage is free once these MMAs have read it (in a pair: in both CTAs)
        if constexpr (kPair) {
          umma_commit_pair(bars + (kStagesG + s) * 8);
          umma_commit_pair(map_to_cta(bars + (kStagesG + s) * 8, 1));
        } else {
          umma_commit(bars + (kStagesG + s) * 8);
        }
      }
      __syncwarp();
    }
    if (lane == 0) {  // all MMAs done: accumulators are final
      if constexpr (kPair) {
        umma_commit_pair(bars + 2 * kStagesG * 8);
        umma_commit_pair(map_to_cta(bars + 2 * kStagesG * 8, 1));
      } else {
        umma_commit(bars + 2 * kStagesG * 8);
      }
    }
    __syncwarp();
    it_base += ksteps;
    }  // fragments
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if constexpr (kPair) cluster_sync_all();  // neither CTA leaves, or frees TMEM, while the other still works
  else __syncthreads();
  if (warp == kProducerWarps) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if constexpr (kPair)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <bool kScaleF16>
__global__ void __launch_bounds__(kGemmThreads, 1)
qgemm_i4_kernel(const GemmParams p) { qgemm_body<false, kScaleF16, false, 1>(p, nullptr); }

template <bool kScaleF16>
__global__ void __launch_bounds__(kGemmThreads, 1)
qgemm_i4_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap x_map) { qgemm_body<false, kScaleF16, true, 2>(p, &x_map); }

// The same kernel over a tiled int8 weight (per-output-channel scales): only the producers'
// weight path differs.  Replaces the reference's large-M linear variants with in-kernel int8
// dequant (the ":wi8" pipeline keys — packages/runtime/src/kernels/weight-storage.ts:82-83,
// geometry from packages/runtime/src/kernels/gemm-geometry.ts:243-267).
template <bool kScaleF16>
__global__ void __launch_bounds__(kGemmThreads, 1)
qgemm_i8_kernel(const GemmParams p) { qgemm_body<true, kScaleF16, false, 1>(p, nullptr); }

template <bool kScaleF16>
__global__ void __launch_bounds__(kGemmThreads, 1)
qgemm_i8_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap x_map) { qgemm_body<true, kScaleF16, true, 2>(p, &x_map); }

// out = bias + sum over the K slices, slices in ascending order (deterministic).
__global__ void __launch_bounds__(256)
qgemm_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ bias, float* __restrict__ out,
                    uint32_t m, uint32_t n, uint32_t splits) {
  const size_t quads = static_cast<size_t>(m) * n / 4;
  const size_t slice = static_cast<size_t>(m) * n;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < quads;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint32_t col = static_cast<uint32_t>((i * 4) % n);
    float4 acc = *reinterpret_cast<const float4*>(partial + i * 4);
    for (uint32_t z = 1; z < splits; ++z) {
      const float4 v = *reinterpret_cast<const float4*>(partial + z * slice + i * 4);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const float4 b = *reinterpret_cast<const float4*>(bias + col);
    acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    *reinterpret_cast<float4*>(out + i * 4) = acc;
  }
}

}  // namespace

bool qgemm_i4_supports(const Weight& w, int x_dtype, uint32_t m) {
  return w.layout == kLayoutTiledI4 && x_dtype == KQ_BF16 && m > 16;
}

bool qgemm_i8_supports(const Weight& w, int x_dtype, uint32_t m) {
  return w.layout == kLayoutTiledI8 && x_dtype == KQ_BF16 && m > 16 && w.k % kBK == 0;
}

namespace {
template <typename Kernel>
cudaError_t launch_gemm_kernel(Kernel kernel, bool* configured, const dim3& grid, size_t smem, cudaStream_t stream,
                               const GemmParams& p) {
  if (!*configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    *configured = true;
  }
  kernel<<<grid, kGemmThreads, smem, stream>>>(p);
  return cudaGetLastError();
}
// The activations [m, k] (bf16, row-major) as a two-dimensional tensor map whose box is one
// stage's tile: 64 columns (128 bytes, the swizzle span) x 256 rows, 128-byte swizzle, rows past
// m read as zero.  The driver's encoder is reached through the runtime (no link against the
// driver library).
cudaError_t encode_activation_map(const void* x, uint32_t m, uint32_t k, CUtensorMap* map) {
  using Encode = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Encode encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess ||
        found != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<Encode>(fn);
  }();
  if (encode == nullptr) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return cudaErrorMisalignedAddress;
  const cuuint64_t dims[2] = {k, m};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * sizeof(__nv_bfloat16)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(kBM)};
  const cuuint32_t element_strides[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, element_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// `resident_pairs`, when given, receives how many pairs of this kernel the device holds at once
// (0 if the query fails) and nothing is launched.
template <typename Kernel>
cudaError_t launch_pair_kernel(Kernel kernel, bool* configured, const dim3& grid, size_t smem, cudaStream_t stream,
                               const GemmParams& p, const CUtensorMap& x_map, int* resident_pairs = nullptr) {
  if (!*configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    *configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (resident_pairs != nullptr) {
    if (cudaOccupancyMaxActiveClusters(resident_pairs, kernel, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      *resident_pairs = 0;
    }
    return cudaSuccess;
  }
  return cudaLaunchKernelEx(&cfg, kernel, p, x_map);
}
}  // namespace

cudaError_t launch_qgemm_i4(const LaunchEnv& env, const LinearTarget& target, const void* x, uint32_t m,
                            int* status_word, int* extra_launches) {
  const Weight& w = *target.w;
  const bool int8 = w.layout == kLayoutTiledI8;
  if (w.layout != kLayoutTiledI4 && !(int8 && w.k % kBK == 0)) return cudaErrorInvalidValue;
  GemmParams p = {};
  p.w = static_cast<const uint8_t*>(w.data);
  p.scale = w.scale;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.bias = target.bias;
  p.out = target.out;
  p.m = m;
  p.n = w.n;
  p.k = w.k;
  p.status = status_word;
  // Three stages of 64 KB, or in the pair form four of 48 KB: the same total.
  const size_t smem = kStagesG * kStageBytes + 1024 + 256;
  // Two or more row tiles: CTA pairs (each pair = two consecutive row tiles of one column tile).
  const bool pair = m > static_cast<uint32_t>(kBM);
  const uint32_t n_tiles = (w.n + kBN - 1) / kBN;
  const uint32_t m_tiles = pair ? (((m + kBM - 1) / kBM + 1u) & ~1u) : (m + kBM - 1) / kBM;
  // Few output tiles: split K over blockIdx.z until the grid covers the machine, as long as a
  // slice keeps at least 8 k-steps and the partial sums fit the context's scratch.
  const uint32_t tiles = n_tiles * m_tiles;
  const uint32_t ksteps_total = w.k / kBK;
  uint32_t splits = 1;
  while (splits < 8 && tiles * splits * 2 <= static_cast<uint32_t>(env.sm_count) && ksteps_total / (splits * 2) >= 8 &&
         static_cast<uint64_t>(splits * 2) * m * w.n * sizeof(float) <= env.workspace_bytes && env.workspace != nullptr)
    splits *= 2;
  p.splits = splits;
  p.ksteps_per_split = (ksteps_total + splits - 1) / splits;
  p.partial = static_cast<float*>(env.workspace);
  // What is remembered per kernel — the shared-memory attribute set, the pairs resident at once —
  // is a property of the device the context runs on: one row per device.
  constexpr int kMaxDevices = 64;
  static bool configured_all[kMaxDevices][8] = {};
  static int resident_all[kMaxDevices][8] = {};  // 0: not asked yet; -1: the query failed
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  bool* configured = configured_all[device];
  int* resident_pairs = resident_all[device];
  cudaError_t e;
  const bool f16 = w.scale_dtype == KQ_F16;
  if (pair) {
    const int which = int8 ? (f16 ? 6 : 7) : (f16 ? 4 : 5);
    alignas(64) CUtensorMap x_map;
    e = encode_activation_map(x, m, w.k, &x_map);
    if (e != cudaSuccess) return e;
    auto launch = [&](const dim3& grid, int* resident) {
      switch (which) {
        case 4: return launch_pair_kernel(qgemm_i4_pair_kernel<true>, &configured[4], grid, smem, env.stream, p, x_map, resident);
        case 5: return launch_pair_kernel(qgemm_i4_pair_kernel<false>, &configured[5], grid, smem, env.stream, p, x_map, resident);
        case 6: return launch_pair_kernel(qgemm_i8_pair_kernel<true>, &configured[6], grid, smem, env.stream, p, x_map, resident);
        default: return launch_pair_kernel(qgemm_i8_pair_kernel<false>, &configured[7], grid, smem, env.stream, p, x_map, resident);
      }
    };
    // Streaming: as many pairs as the device holds at once, each given one contiguous run of
    // (pair tile, k-step) units, so that no SM waits for a last, nearly empty wave of tiles.  The
    // pieces of tiles that two pairs share go through the context's scratch and are added by the
    // tile's first pair.  Taken when the last wave of whole tiles would leave 15 % or more of
    // the machine's time unused and a run is at least one tile long (a tile then has at most
    // two owners); measured slower than whole tiles otherwise.  A pure function of the shapes.
    if (resident_pairs[which] == 0) {
      e = launch(dim3(2, 1, 1), &resident_pairs[which]);
      if (e != cudaSuccess) return e;
      if (resident_pairs[which] <= 0) resident_pairs[which] = -1;
    }
    const uint32_t pair_tiles = n_tiles * (m_tiles / 2);
    const uint32_t stream_pairs = static_cast<uint32_t>(std::max(resident_pairs[which], 0));
    const bool unbalanced = stream::worth_streaming(pair_tiles, stream_pairs, ksteps_total);
    const uint64_t slot_bytes = static_cast<uint64_t>(stream_pairs) * 2 * kBM * kBN * sizeof(float);
    if (unbalanced && env.workspace != nullptr && slot_bytes <= env.workspace_bytes && env.counters != nullptr &&
        stream_pairs * 2 <= env.counter_count) {
      p.splits = 1;
      p.stream_pairs = stream_pairs;
      p.pair_tiles = pair_tiles;
      p.m_pairs = m_tiles / 2;
      p.slots = static_cast<float*>(env.workspace);
      p.flags = env.counters;
      e = cudaMemsetAsync(p.flags, 0, stream_pairs * 2 * sizeof(unsigned int), env.stream);  // flags a failed launch may have left up
      if (e != cudaSuccess) return e;
      return launch(dim3(stream_pairs * 2, 1, 1), nullptr);
    }
    // x walks m in whole pairs (a CTA past the last row computes on zero-filled rows and stores nothing), y walks n
    e = launch(dim3(m_tiles, n_tiles, splits), nullptr);
  } else {
    const dim3 grid(n_tiles, m_tiles, splits);
    if (int8)
      e = f16 ? launch_gemm_kernel(qgemm_i8_kernel<true>, &configured[2], grid, smem, env.stream, p)
              : launch_gemm_kernel(qgemm_i8_kernel<false>, &configured[3], grid, smem, env.stream, p);
    else
      e = f16 ? launch_gemm_kernel(qgemm_i4_kernel<true>, &configured[0], grid, smem, env.stream, p)
              : launch_gemm_kernel(qgemm_i4_kernel<false>, &configured[1], grid, smem, env.stream, p);
  }
  if (e != cudaSuccess || splits == 1) return e;
  const size_t quads = static_cast<size_t>(m) * w.n / 4;
  const int rgrid = static_cast<int>(std::min<size_t>((quads + 255) / 256, static_cast<size_t>(env.sm_count) * 8));
  qgemm_reduce_kernel<<<rgrid, 256, 0, env.stream>>>(p.partial, p.bias, p.out, m, w.n, splits);
  if (extra_launches) *extra_launches += 1;
  return cudaGetLastError();
}

}  // namespace kq
