// qgemm_i4_x32 — the prefill GEMM for f32 and binary16 activations:
//   out[m, n] = x[m, k] . W[n, k]^T + bias,  m > 16, W in the tiled int4 / group-32 layout.
//
// The reference's large-M linear variants compute in f32 (linear:v2:f32:reg128x128r8x8w16 —
// packages/runtime/src/kernels/gemm-geometry.ts:243-267).  The tensor cores take 16-bit inputs,
// so both operands are carried as TWO bf16 numbers and the three significant products are
// accumulated in f32:
//     x = x_hi + x_lo          (x_hi = RNE_bf16(x), x_lo = RNE_bf16(x - x_hi): 16 significant bits;
//                               exact for binary16 activations, whose 11 bits fit)
//     w = w_hi + w_lo          (w = fround((u - 8) * s), the reference's dequantised value;
//                               exact when the scale is a binary16 number: 15 bits)
//     x . w ~ x_hi w_hi + x_hi w_lo + x_lo w_hi        (the dropped x_lo w_lo is 2^-16 of a term)
// Per element that leaves a relative error of 2^-17 (f32 activations) against 2^-9 when the
// operands are rounded to bf16 once (kq_qgemm_i4.cu).  The result contract is the decode path's
// rtol with atol = 4e-5 * max(1, rms(ref)).
//
//   CTA tile 128 (m) x 256 (n), k-step 64, two shared-memory stages of 96 KB:
//     [x_hi 128 x 64][x_lo 128 x 64][w_hi 256 x 64][w_lo 256 x 64], each K-major, 128-byte swizzled.
//   warps 0-15 producers: cp.async the two activation tiles (split once per launch by
//              split_x_kernel into the context's scratch) and dequantise one 16-row chunk each
//              into the two weight tiles; afterwards they drain the accumulator.
//   warp 16    one thread issues three tcgen05.mma (M 128 x N 256 x K 16) per k16 slice into ONE
//              128 x 256 f32 accumulator (256 tensor-memory columns) and commits each stage back.
//   Few output tiles: K is split over blockIdx.z into partial sums that x32_reduce_kernel adds
//   in slice order.  Activations are processed in row panels that fit the scratch.
// Every mbarrier wait is bounded (status word + CTA-wide abort flag), as in kq_qgemm_i4.cu.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

#include "kq_common.cuh"
#include "kq_internal.h"
#include "kq_umma.cuh"

namespace kq {
namespace {

using namespace umma;

constexpr int kXM = 128, kXN = 256, kXK = 64, kXStages = 2;
constexpr int kXProducerWarps = 16;
constexpr int kXThreads = kXProducerWarps * 32 + 32;
constexpr uint32_t kXATile = kXM * kXK * 2;                 // 16 KB, one of x_hi / x_lo
constexpr uint32_t kXBTile = kXN * kXK * 2;                 // 32 KB, one of w_hi / w_lo
constexpr uint32_t kXStage = 2 * kXATile + 2 * kXBTile;     // 96 KB
constexpr uint32_t kXTmemCols = 256;
constexpr int kXPieces = (2 * kXM * 8) / (kXProducerWarps * 32);  // 16-byte activation pieces per thread and k-step

struct X32Params {
  const uint8_t* w;
  const __nv_bfloat16* x_hi;
  const __nv_bfloat16* x_lo;
  const float* bias;
  float* out;
  uint32_t m, n, k;
  int* status;
  uint32_t ksteps_per_split, splits;
  float* partial;  // [splits][m][n] when splits > 1
};

// x -> (RNE_bf16(x), RNE_bf16(x - RNE_bf16(x))), eight elements per thread.
template <typename XT>
__global__ void __launch_bounds__(256)
split_x_kernel(const XT* __restrict__ x, uint64_t octets, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
  for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < octets; i += static_cast<uint64_t>(gridDim.x) * 256ull) {
    float v[8];
    if constexpr (std::is_same<XT, float>::value) {
      const float4 a = reinterpret_cast<const float4*>(x)[2 * i], b = reinterpret_cast<const float4*>(x)[2 * i + 1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
      const uint4 raw = reinterpret_cast<const uint4*>(x)[i];
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
      }
    }
    uint4 oh, ol;
    uint32_t* ph = reinterpret_cast<uint32_t*>(&oh);
    uint32_t* pl = reinterpret_cast<uint32_t*>(&ol);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      const float2 back = __bfloat1622float2(h2);
      const __nv_bfloat162 l2 = __floats2bfloat162_rn(v[2 * j] - back.x, v[2 * j + 1] - back.y);
      ph[j] = *reinterpret_cast<const uint32_t*>(&h2);
      pl[j] = *reinterpret_cast<const uint32_t*>(&l2);
    }
    reinterpret_cast<uint4*>(hi)[i] = oh;
    reinterpret_cast<uint4*>(lo)[i] = ol;
  }
}

// 8 nibbles of one word -> 8 dequantised values w = fround((u - 8) * s) as bf16 pairs (hi, lo):
// the exact integer-to-float trick of dequant8_bf16, then w_hi = RNE_bf16(w), w_lo = RNE_bf16(w - w_hi).
__device__ __forceinline__ void dequant8_split(uint32_t word, float s, uint4& hi, uint4& lo) {
  const float s1 = s * 0.0625f, s2 = s * 0.00390625f, s3 = s * 0.000244140625f;
  const uint32_t top = word >> 16;
  float v[8];
  v[0] = (__uint_as_float((word & 0x000Fu) | 0x4B000000u) - 8388616.0f) * s;
  v[1] = (__uint_as_float((word & 0x00F0u) | 0x4B000000u) - 8388736.0f) * s1;
  v[2] = (__uint_as_float((word & 0x0F00u) | 0x4B000000u) - 8390656.0f) * s2;
  v[3] = (__uint_as_float((word & 0xF000u) | 0x4B000000u) - 8421376.0f) * s3;
  v[4] = (__uint_as_float((top & 0x000Fu) | 0x4B000000u) - 8388616.0f) * s;
  v[5] = (__uint_as_float((top & 0x00F0u) | 0x4B000000u) - 8388736.0f) * s1;
  v[6] = (__uint_as_float((top & 0x0F00u) | 0x4B000000u) - 8390656.0f) * s2;
  v[7] = (__uint_as_float((top & 0xF000u) | 0x4B000000u) - 8421376.0f) * s3;
  uint32_t* ph = reinterpret_cast<uint32_t*>(&hi);
  uint32_t* pl = reinterpret_cast<uint32_t*>(&lo);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    const float2 back = __bfloat1622float2(h2);
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(v[2 * j] - back.x, v[2 * j + 1] - back.y);
    ph[j] = *reinterpret_cast<const uint32_t*>(&h2);
    pl[j] = *reinterpret_cast<const uint32_t*>(&l2);
  }
}

template <bool kScaleF16>
__global__ void __launch_bounds__(kXThreads, 1)
qgemm_i4_x32_kernel(const X32Params p) {
  constexpr uint32_t kScaleBytes = kScaleF16 ? 2u : 4u;
  constexpr uint32_t kCB = kChunkWeightBytes + 32u * kScaleBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t raw_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
  const uint32_t tiles = (raw_base + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  // barriers behind the stages: full[2], empty[2], accumulator; then the TMEM base and the abort flag
  const uint32_t bars = tiles + kXStages * kXStage;
  const uint32_t tmem_slot = bars + 64;
  uint8_t* generic_base = smem_raw + (tiles - raw_base);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(generic_base + kXStages * kXStage + 72);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + kXStages * kXStage + 64);

  const uint32_t n0 = blockIdx.x * kXN, m0 = blockIdx.y * kXM;
  const uint32_t ks_begin = blockIdx.z * p.ksteps_per_split;
  const uint32_t ks_end = min(ks_begin + p.ksteps_per_split, p.k / kXK);
  const uint32_t ksteps = ks_end - ks_begin;
  const uint32_t chunks_per_row = p.k / kChunkK;

  if (warp == kXProducerWarps) {
    if (lane == 0) {
      for (int s = 0; s < kXStages; ++s) {
        mbar_init(bars + s * 8, kXProducerWarps * 32);  // full: every producer thread arrives
        mbar_init(bars + (kXStages + s) * 8, 1);        // empty: one tcgen05.commit
      }
      mbar_init(bars + 2 * kXStages * 8, 1);            // accumulator complete
      *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kXTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp < kXProducerWarps) {
    // ---------------- producers ----------------
    const uint32_t tid = threadIdx.x;
    const uint32_t g = lane >> 2, t = lane & 3u;
    // the lane's word of the warp's chunk (row block n0 / 16 + warp) and its scales, one k-step ahead
    const uint32_t row0 = n0 + warp * 16u;
    const bool chunk_live = row0 < p.n;
    const uint8_t* chunk_ptr = p.w + (static_cast<size_t>(row0 >> 4) * chunks_per_row + ks_begin) * kCB + lane * 16;
    const uint32_t scale_off = kChunkWeightBytes - lane * 16 + g * (kScaleF16 ? 8u : 16u);
    uint4 wq_next = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);  // u = 8 -> value 0
    typename std::conditional<kScaleF16, uint2, uint4>::type sc_next;
    auto fetch_weights = [&](uint32_t ks) {
      wq_next = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
      if constexpr (kScaleF16) sc_next = make_uint2(0, 0);
      else sc_next = make_uint4(0, 0, 0, 0);
      if (chunk_live && ks < ksteps) {
        wq_next = *reinterpret_cast<const uint4*>(chunk_ptr);
        if constexpr (kScaleF16) sc_next = *reinterpret_cast<const uint2*>(chunk_ptr + scale_off);
        else sc_next = *reinterpret_cast<const uint4*>(chunk_ptr + scale_off);
        chunk_ptr += kCB;
      }
    };
    // the thread's activation pieces: 2 tiles x 128 rows x 8 pieces of 16 B per k-step
    const __nv_bfloat16* a_src[kXPieces];
    uint32_t a_dst[kXPieces], a_bytes[kXPieces];
#pragma unroll
    for (int i = 0; i < kXPieces; ++i) {
      const uint32_t piece = tid + i * (kXProducerWarps * 32u);
      const uint32_t which = piece >> 10, r = (piece >> 3) & 127u, c = piece & 7u;
      const bool in_range = m0 + r < p.m;
      a_src[i] = (which ? p.x_lo : p.x_hi) + static_cast<size_t>(in_range ? m0 + r : 0) * p.k + ks_begin * kXK + c * 8;
      a_dst[i] = which * kXATile + swz(r, c);
      a_bytes[i] = in_range ? 16u : 0u;
    }
    fetch_weights(0);
    for (uint32_t ks = 0; ks < ksteps; ++ks) {
      const uint32_t s = ks % kXStages, phase = (ks / kXStages) & 1u;
      wait_bounded(bars + (kXStages + s) * 8, phase ^ 1u, abort_flag, p.status, 11);
      const uint32_t a_tile = tiles + s * kXStage, b_hi = a_tile + 2 * kXATile, b_lo = b_hi + kXBTile;
#pragma unroll
      for (int i = 0; i < kXPieces; ++i) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a_tile + a_dst[i]), "l"(a_src[i]), "r"(a_bytes[i])
                     : "memory");
        a_src[i] += kXK;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      const uint4 wq = wq_next;
      float sc[4];
      if constexpr (kScaleF16) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&sc_next.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&sc_next.y));
        sc[0] = a.x; sc[1] = a.y; sc[2] = b.x; sc[3] = b.y;
      } else {
        sc[0] = __uint_as_float(sc_next.x); sc[1] = __uint_as_float(sc_next.y);
        sc[2] = __uint_as_float(sc_next.z); sc[3] = __uint_as_float(sc_next.w);
      }
      fetch_weights(ks + 1);
      // words: row g grp 0 | row g+8 grp 0 | row g grp 1 | row g+8 grp 1; the lane's 8 nibbles of a
      // group are 16-byte piece t (group 0) or 4 + t (group 1) of the 128-byte tile row.  Odd g
      // stores group 1 first, so the lanes of a shared-memory phase hit different columns.
      const uint32_t r_a = warp * 16u + g, r_b = r_a + 8u;
      const bool odd = (g & 1u) != 0;
      const uint32_t off_a0 = swz(r_a, t), off_a1 = swz(r_a, 4u + t), off_b0 = swz(r_b, t), off_b1 = swz(r_b, 4u + t);
      uint4 h0, l0, h1, l1;
      dequant8_split(wq.x, sc[0], h0, l0);
      dequant8_split(wq.z, sc[2], h1, l1);
      sts128(b_hi + (odd ? off_a1 : off_a0), odd ? h1 : h0);
      sts128(b_lo + (odd ? off_a1 : off_a0), odd ? l1 : l0);
      sts128(b_hi + (odd ? off_a0 : off_a1), odd ? h0 : h1);
      sts128(b_lo + (odd ? off_a0 : off_a1), odd ? l0 : l1);
      dequant8_split(wq.y, sc[1], h0, l0);
      dequant8_split(wq.w, sc[3], h1, l1);
      sts128(b_hi + (odd ? off_b1 : off_b0), odd ? h1 : h0);
      sts128(b_lo + (odd ? off_b1 : off_b0), odd ? l1 : l0);
      sts128(b_hi + (odd ? off_b0 : off_b1), odd ? h0 : h1);
      sts128(b_lo + (odd ? off_b0 : off_b1), odd ? l0 : l1);
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
      mbar_arrive(bars + s * 8);
    }
    // ---------------- epilogue: accumulator -> out ----------------
    wait_bounded(bars + 2 * kXStages * 8, 0, abort_flag, p.status, 13);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // a warp may only touch the TMEM lane quarter warp % 4; the four warps of a quarter take 64
    // columns each
    const uint32_t quarter = warp & 3u, group = warp >> 2;
    const uint32_t row = m0 + quarter * 32u + lane;
    float* scratch = reinterpret_cast<float*>(generic_base) + warp * (32u * 36u);
#pragma unroll 1
    for (uint32_t cb = group * 2u; cb < group * 2u + 2u; ++cb) {
      uint32_t v[32];
      const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + cb * 32u;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
          "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
            "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
            "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
            "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      // through shared memory (the stage buffers are free by now) so that every row leaves as one
      // coalesced 128-byte store
      const uint32_t col0 = n0 + cb * 32u;
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(scratch + lane * 36u + j) =
            make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      __syncwarp();
      const bool final_sum = p.splits == 1;
      const uint32_t col = col0 + lane;
      if (col < p.n) {
        const float b = final_sum ? p.bias[col] : 0.0f;
        const uint32_t row_first = row - lane;
        float* dst = (final_sum ? p.out : p.partial + static_cast<size_t>(blockIdx.z) * p.m * p.n) + col;
        const uint32_t rows_here = row_first < p.m ? min(32u, p.m - row_first) : 0u;
        for (uint32_t rr = 0; rr < rows_here; ++rr)
          dst[static_cast<size_t>(row_first + rr) * p.n] = scratch[rr * 36u + lane] + b;
      }
    }
  } else {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t kIdesc = umma_idesc(128, kXN);
    for (uint32_t ks = 0; ks < ksteps; ++ks) {
      const uint32_t s = ks % kXStages, phase = (ks / kXStages) & 1u;
      const bool ok = wait_bounded(bars + s * 8, phase, abort_flag, p.status, 12);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint32_t a_hi = tiles + s * kXStage, a_lo = a_hi + kXATile, b_hi = a_hi + 2 * kXATile, b_lo = b_hi + kXBTile;
        if (ok) {
#pragma unroll
          for (uint32_t kk = 0; kk < kXK / 16; ++kk) {
            const uint64_t dah = umma_desc(a_hi + kk * 32u), dal = umma_desc(a_lo + kk * 32u);
            const uint64_t dbh = umma_desc(b_hi + kk * 32u), dbl = umma_desc(b_lo + kk * 32u);
            umma_bf16(tmem_base, dah, dbh, kIdesc, (ks | kk) != 0 ? 1u : 0u);
            umma_bf16(tmem_base, dah, dbl, kIdesc, 1u);
            umma_bf16(tmem_base, dal, dbh, kIdesc, 1u);
          }
        }
        umma_commit(bars + (kXStages + s) * 8);  // the stage is free once these MMAs have read it
      }
      __syncwarp();
    }
    if (lane == 0) umma_commit(bars + 2 * kXStages * 8);  // all MMAs done: the accumulator is final
    __syncwarp();
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kXProducerWarps) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kXTmemCols) : "memory");
  }
}

// out = bias + sum over the K slices, slices in ascending order (deterministic).
__global__ void __launch_bounds__(256)
x32_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ bias, float* __restrict__ out, uint32_t m,
                  uint32_t n, uint32_t splits) {
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

template <typename XT>
cudaError_t launch_x32(const LaunchEnv& env, const LinearTarget& target, const XT* x, uint32_t m, int* status_word,
                       int* launches) {
  const Weight& w = *target.w;
  const uint32_t ksteps_total = w.k / kXK;
  const size_t smem = kXStages * kXStage + 1024 + 256;
  if (env.workspace == nullptr) return cudaErrorMemoryAllocation;
  // The tensor core's f32 accumulation loses precision with the length of the chain (as adds that
  // truncate would): over a chain of c accumulating MMAs the sum drifts by about c * 2^-24 of its
  // magnitude (measured: 3.5e-4 of the output's rms over
  // k = 14336 in one chain, 2,688 MMAs).  A chain therefore covers at most 32 k-steps (2048 k, 384
  // MMAs); longer K is split over blockIdx.z and the slices are added in IEEE f32 by
  // x32_reduce_kernel, whatever the number of tiles.
  const uint32_t chain_splits = (ksteps_total + 31) / 32;
  // row panels: [x_hi | x_lo] of a panel, then the partial sums of a split launch, fit the scratch
  const uint64_t row_bytes = static_cast<uint64_t>(w.k) * 2 * sizeof(__nv_bfloat16);
  const uint64_t per_row = row_bytes + (chain_splits > 1 ? static_cast<uint64_t>(chain_splits) * w.n * sizeof(float) : 0);
  if (per_row * 32 > env.workspace_bytes) return cudaErrorMemoryAllocation;
  uint32_t panel = static_cast<uint32_t>(std::min<uint64_t>(m, env.workspace_bytes / per_row));
  if (panel >= static_cast<uint32_t>(kXM)) panel = panel / kXM * kXM;
  for (uint32_t r0 = 0; r0 < m; r0 += panel) {
    const uint32_t pm = std::min(panel, m - r0);
    __nv_bfloat16* hi = static_cast<__nv_bfloat16*>(env.workspace);
    __nv_bfloat16* lo = hi + static_cast<size_t>(pm) * w.k;
    float* partial = reinterpret_cast<float*>(lo + static_cast<size_t>(pm) * w.k);
    const uint64_t partial_room = env.workspace_bytes - static_cast<uint64_t>(pm) * row_bytes;
    const uint64_t octets = static_cast<uint64_t>(pm) * w.k / 8;
    const int sgrid = static_cast<int>(std::min<uint64_t>((octets + 255) / 256, static_cast<uint64_t>(env.sm_count) * 16));
    split_x_kernel<XT><<<sgrid, 256, 0, env.stream>>>(x + static_cast<size_t>(r0) * w.k, octets, hi, lo);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    X32Params p = {};
    p.w = static_cast<const uint8_t*>(w.data);
    p.x_hi = hi;
    p.x_lo = lo;
    p.bias = target.bias;
    p.out = target.out + static_cast<size_t>(r0) * w.n;
    p.m = pm;
    p.n = w.n;
    p.k = w.k;
    p.status = status_word;
    const uint32_t tiles = ((w.n + kXN - 1) / kXN) * ((pm + kXM - 1) / kXM);
    uint32_t splits = chain_splits;
    while (splits < 8 && tiles * splits * 2 <= static_cast<uint32_t>(env.sm_count) && ksteps_total / (splits * 2) >= 8 &&
           static_cast<uint64_t>(splits * 2) * pm * w.n * sizeof(float) <= partial_room)
      splits *= 2;
    p.splits = splits;
    p.ksteps_per_split = (ksteps_total + splits - 1) / splits;
    p.partial = partial;
    const dim3 grid((w.n + kXN - 1) / kXN, (pm + kXM - 1) / kXM, splits);
    if (w.scale_dtype == KQ_F16) {
      static PerDevice<bool> configured_on;
      bool* configured = configured_on.slot();
      if (configured == nullptr) return cudaErrorInvalidDevice;
      if (!*configured) {
        e = cudaFuncSetAttribute(qgemm_i4_x32_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        *configured = true;
      }
      qgemm_i4_x32_kernel<true><<<grid, kXThreads, smem, env.stream>>>(p);
    } else {
      static PerDevice<bool> configured_on;
      bool* configured = configured_on.slot();
      if (configured == nullptr) return cudaErrorInvalidDevice;
      if (!*configured) {
        e = cudaFuncSetAttribute(qgemm_i4_x32_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        *configured = true;
      }
      qgemm_i4_x32_kernel<false><<<grid, kXThreads, smem, env.stream>>>(p);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) *launches += 2;
    if (splits > 1) {
      const size_t quads = static_cast<size_t>(pm) * w.n / 4;
      const int rgrid = static_cast<int>(std::min<size_t>((quads + 255) / 256, static_cast<size_t>(env.sm_count) * 8));
      x32_reduce_kernel<<<rgrid, 256, 0, env.stream>>>(partial, p.bias, p.out, pm, w.n, splits);
      e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      if (launches) *launches += 1;
    }
  }
  return cudaSuccess;
}

}  // namespace

bool qgemm_i4_x32_supports(const Weight& w, int x_dtype, uint32_t m, uint64_t workspace_bytes) {
  if (w.layout != kLayoutTiledI4 || (x_dtype != KQ_F32 && x_dtype != KQ_F16) || m <= 16 || w.n == 0) return false;
  // 32 rows of the split activations and of the partial sums must fit the scratch (launch_x32)
  const uint64_t chain_splits = (w.k / kXK + 31) / 32;
  const uint64_t per_row = static_cast<uint64_t>(w.k) * 4 + (chain_splits > 1 ? chain_splits * w.n * sizeof(float) : 0);
  return per_row * 32 <= workspace_bytes;
}

cudaError_t launch_qgemm_i4_x32(const LaunchEnv& env, const LinearTarget& target, const void* x, int x_dtype, uint32_t m,
                                int* status_word, int* launches) {
  if (!qgemm_i4_x32_supports(*target.w, x_dtype, m, env.workspace ? env.workspace_bytes : 0)) return cudaErrorInvalidValue;
  if (x_dtype == KQ_F32) return launch_x32<float>(env, target, static_cast<const float*>(x), m, status_word, launches);
  return launch_x32<__half>(env, target, static_cast<const __half*>(x), m, status_word, launches);
}

}  // namespace kq
