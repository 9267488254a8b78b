// Building blocks shared by the tensor-core int4 GEMV kernels (the per-launch kernel and the
// persistent plan kernel): the binary16-subnormal nibble trick, MMA wrappers, and the
// staging of activations into the k-order the nibble pairs come out in.
#pragma once

#include <type_traits>

#include "kq_common.cuh"

namespace kq {

constexpr float kUnscale = 16777216.0f;  // 2^24: undoes the subnormal encoding of the nibbles

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

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

// kFromL2: read through L2 (ld.global.cg).  Needed when the activations were written
// by another CTA of the SAME kernel, which the non-coherent L1 may not have seen.
template <typename XT, bool kFromL2 = false>
__device__ __forceinline__ void load_x8(const XT* p, float (&v)[8]) {
  if constexpr (std::is_same<XT, float>::value) {
    const float4 a = kFromL2 ? __ldcg(reinterpret_cast<const float4*>(p)) : reinterpret_cast<const float4*>(p)[0];
    const float4 b = kFromL2 ? __ldcg(reinterpret_cast<const float4*>(p) + 1) : reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = kFromL2 ? __ldcg(reinterpret_cast<const uint4*>(p)) : *reinterpret_cast<const uint4*>(p);
    const uint32_t parts[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same<XT, __half>::value) {
        v[2 * i] = half_bits_to_float(parts[i] & 0xFFFFu);
        v[2 * i + 1] = half_bits_to_float(parts[i] >> 16);
      } else {
        v[2 * i] = __uint_as_float(parts[i] << 16);
        v[2 * i + 1] = __uint_as_float(parts[i] & 0xFFFF0000u);
      }
    }
  }
}
// ---- power-of-two pre-scale of the activations -------------------------------------------
// binary16 has a narrow exponent range, f32 activations do not.  Before an activation is split
// into binary16 parts it is multiplied by 2^e, with e chosen from the largest magnitude of the
// values that share it (a 32-k scale group of one activation row, or a whole activation row),
// so that this maximum lands in [2^13, 2^14).  The multiplication is exact, the matching
// 2^-e is applied in f32 to the group's (or row's) partial sum, and the result no longer
// depends on the magnitude of x: there is neither an upper limit at 65504 nor an absolute
// error floor at the binary16 subnormal grid (the parts then resolve 2^-37 of the maximum,
// 2^-33 for the odd positions that are stored divided by 16).
// A maximum of zero or a non-finite one leaves the values as they are (e = 0): Inf and NaN
// reach the MMA unchanged and make the outputs of that activation row non-finite, as they do
// in an f32 multiply-add.
struct Pow2 {
  float scale;  // 2^e
  float inv;    // 2^-e
};
__device__ __forceinline__ Pow2 pow2_prescale(float amax) {
  const uint32_t bits = __float_as_uint(amax) & 0x7fffffffu;
  int e = 0;
  if (bits != 0u && bits < 0x7f800000u) {
    e = 13 + 127 - static_cast<int>(bits >> 23);  // subnormal maxima count as 2^-127
    e = max(-114, min(126, e));
  }
  Pow2 r;
  r.scale = __uint_as_float(static_cast<uint32_t>(e + 127) << 23);
  r.inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
  return r;
}
__device__ __forceinline__ float absmax8(const float (&v)[8]) {
  float a = fabsf(v[0]);
#pragma unroll
  for (int e = 1; e < 8; ++e) a = fmaxf(a, fabsf(v[e]));
  // fmaxf drops NaN operands; an Inf is enough to switch the pre-scale off, and a NaN next to
  // finite values is staged as NaN whatever the scale is
  return a;
}

// Stages groups [group0, group0 + groups) of x into shared memory.
//   xs   : [local group][active columns][32 halfs]; activation row r occupies column r
//          (binary16 input) or columns 2r (hi) and 2r+1 (lo).  The 8 values of each
//          k-octet are stored in the order 0,4,1,5,2,6,3,7, and the odd ones (1,3,5,7)
//          are stored divided by 16: their nibbles reach the MMA as u * 2^-20 instead
//          of u * 2^-24.  Every value is pre-scaled by the 2^e of its (row, group), see above.
//   corr : kPerGroup  : [local group][kCorrStride] float2; entry r = { c, 2^-e } of that
//                       (row, group), c = -8 * 2^-24 * 2^-e * (sum of the group's x of activation
//                       row r, as staged): a group's partial sum is fma(mma sum, 2^-e, c)
//          !kPerGroup : [local group][kCorrStride] f32, the first of the two only; the
//                       caller passes one scale per activation row in row_scale
// Four consecutive threads share one (group, row): each converts one octet.
// kBatch: octets a thread loads before it converts any (one memory round trip per batch, at
// the price of 8 registers per octet held).
//   lo_offset != 0 selects the split layout: activation row r occupies column r, its hi part at
//          byte offset 0 of the group and its lo part lo_offset bytes further on.
// Converts ONE k-octet (8 consecutive activations of one row, already in registers as f32) and
// stores it; the four threads of a (group, row) call this together (the shuffles below run over
// whole warps, so every lane of a warp must make the call, `valid` or not).
template <bool kHasLo, int kCorrStride, bool kPerGroup>
__device__ __forceinline__ void stage_octet(const float (&v)[8], bool valid, uint32_t q, uint32_t row, uint32_t lg,
                                            uint8_t* xs, uint32_t xs_stride, float* corr, uint32_t lo_offset,
                                            const float* row_scale) {
  Pow2 ps;
  if constexpr (kPerGroup) {
    float amax = absmax8(v);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    ps = pow2_prescale(amax);
  } else {
    ps.scale = valid ? row_scale[row] : 1.0f;
    ps.inv = 1.0f;
  }
  uint4 hi4 = make_uint4(0, 0, 0, 0), lo4 = make_uint4(0, 0, 0, 0);
  float sum = 0.0f;
  if (valid) {
    __half h[8], l[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float staged = v[e] * ((e & 1) ? ps.scale * 0.0625f : ps.scale);
      const float back = (e & 1) ? 16.0f : 1.0f;
      h[e] = __float2half_rn(staged);
      const float hf = __half2float(h[e]);
      if constexpr (kHasLo) {
        l[e] = __float2half_rn(staged - hf);
        sum = fmaf(hf + __half2float(l[e]), back, sum);
      } else {
        sum = fmaf(hf, back, sum);
      }
    }
    hi4 = make_uint4(pack_half2(h[0], h[4]), pack_half2(h[1], h[5]), pack_half2(h[2], h[6]), pack_half2(h[3], h[7]));
    if constexpr (kHasLo)
      lo4 = make_uint4(pack_half2(l[0], l[4]), pack_half2(l[1], l[5]), pack_half2(l[2], l[6]), pack_half2(l[3], l[7]));
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  if (valid) {
    const uint32_t col = (kHasLo && lo_offset == 0) ? 2 * row : row;
    const uint32_t off = lg * xs_stride + col * 64 + q * 16;
    *reinterpret_cast<uint4*>(xs + off) = hi4;
    if constexpr (kHasLo) *reinterpret_cast<uint4*>(xs + off + (lo_offset == 0 ? 64u : lo_offset)) = lo4;
    if (q == 0) {
      if constexpr (kPerGroup)
        reinterpret_cast<float2*>(corr)[lg * kCorrStride + row] = make_float2(sum * (-8.0f / kUnscale) * ps.inv, ps.inv);
      else
        corr[lg * kCorrStride + row] = sum * (-8.0f / kUnscale);
    }
  }
}

template <typename XT, bool kHasLo, int kCorrStride, bool kFromL2 = false, int kBatch = 1, bool kPerGroup = true>
__device__ __forceinline__ void stage_x(const XT* __restrict__ x, uint32_t m, uint32_t k,
                                        uint32_t group0, uint32_t groups, uint8_t* xs,
                                        uint32_t xs_stride, float* corr, uint32_t lo_offset = 0,
                                        const float* row_scale = nullptr) {
  const uint32_t items = groups * m * 4;
  const uint32_t items_padded = (items + 31u) & ~31u;  // whole warps run the shuffles
  for (uint32_t base = threadIdx.x; base < items_padded; base += blockDim.x * kBatch) {
    float v[kBatch][8];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const uint32_t item = base + b * blockDim.x;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[b][e] = 0.0f;
      if (item < items) {
        const uint32_t rest = item >> 2;
        const uint32_t row = rest % m, lg = rest / m;
        load_x8<XT, kFromL2>(x + static_cast<size_t>(row) * k + (static_cast<size_t>(group0 + lg) << 5) + ((item & 3u) << 3),
                             v[b]);
      }
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const uint32_t item = base + b * blockDim.x;
      if (item >= items_padded) break;  // warp-uniform
      const uint32_t rest = item >> 2;
      stage_octet<kHasLo, kCorrStride, kPerGroup>(v[b], item < items, item & 3u, rest % m, rest / m, xs, xs_stride,
                                                  corr, lo_offset, row_scale);
    }
  }
}

// The same with an rms_norm in front (the whole activation block, group0 = 0):
//   v = (x * rsqrt(mean_row(x^2) + eps)) * weight[k]        (packages/runtime/src/kernels/rms-norm.ts:60-90)
// is what gets staged.  The sum of squares of a row is taken over the CTA: every thread adds
// the squares of its own octets in ascending order, a warp adds its lanes with the shuffle
// tree, and the warps' sums are added in warp order, so every CTA that stages the same x
// computes the same bits.  `red` is [warps][m] floats of shared memory (`inv` is unused).
// When the block fits one round (items <= threads * kBatch, every decode shape) the octets
// stay in registers between the two passes; otherwise x is read a second time.
template <typename XT, bool kHasLo, int kCorrStride, bool kFromL2, int kBatch, int kMaxRows>
__device__ __forceinline__ void stage_x_rms_norm(const XT* __restrict__ x, const float* __restrict__ weight, float eps,
                                                 uint32_t m, uint32_t k, uint8_t* xs, uint32_t xs_stride, float* corr,
                                                 float* red, float* inv) {
  const uint32_t groups = k >> 5;
  const uint32_t items = groups * m * 4;
  const uint32_t items_padded = (items + 31u) & ~31u;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
  const bool one_round = items_padded <= blockDim.x * kBatch;
  float v[kBatch][8];
  float sq[kMaxRows];  // m <= kMaxRows
#pragma unroll
  for (int r = 0; r < kMaxRows; ++r) sq[r] = 0.0f;
  for (uint32_t base = threadIdx.x; base < items_padded; base += blockDim.x * kBatch) {
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const uint32_t item = base + b * blockDim.x;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[b][e] = 0.0f;
      if (item < items) {
        const uint32_t rest = item >> 2;
        const uint32_t row = rest % m, lg = rest / m;
        load_x8<XT, kFromL2>(x + static_cast<size_t>(row) * k + (static_cast<size_t>(lg) << 5) + ((item & 3u) << 3), v[b]);
        float s = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) s = fmaf(v[b][e], v[b][e], s);
#pragma unroll
        for (int r = 0; r < kMaxRows; ++r)
          if (static_cast<uint32_t>(r) == row) sq[r] += s;
      }
    }
  }
  // the norm weights of the thread's first octet travel while the sums of squares meet
  float wv0[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (threadIdx.x < items) {
    const uint32_t lg0 = (threadIdx.x >> 2) / m, q0 = threadIdx.x & 3u;
    const float4 w0 = __ldg(reinterpret_cast<const float4*>(weight + (lg0 << 5) + (q0 << 3)));
    const float4 w1 = __ldg(reinterpret_cast<const float4*>(weight + (lg0 << 5) + (q0 << 3) + 4));
    wv0[0] = w0.x; wv0[1] = w0.y; wv0[2] = w0.z; wv0[3] = w0.w;
    wv0[4] = w1.x; wv0[5] = w1.y; wv0[6] = w1.z; wv0[7] = w1.w;
  }
#pragma unroll
  for (int r = 0; r < kMaxRows; ++r) {
    if (static_cast<uint32_t>(r) < m) {  // uniform
      const float total = warp_sum(sq[r]);
      if (lane == 0) red[warp * m + r] = total;
    }
  }
  __syncthreads();
  (void)inv;
  for (uint32_t base = threadIdx.x; base < items_padded; base += blockDim.x * kBatch) {
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const uint32_t item = base + b * blockDim.x;
      if (item >= items_padded) break;  // warp-uniform
      const bool valid = item < items;
      const uint32_t rest = item >> 2;
      const uint32_t row = rest % m, lg = rest / m, q = item & 3u;
      if (valid) {
        if (!one_round)
          load_x8<XT, kFromL2>(x + static_cast<size_t>(row) * k + (static_cast<size_t>(lg) << 5) + (q << 3), v[b]);
        // every thread adds the warps' sums of its row itself, in warp order: the same bits in
        // every thread and in every CTA
        float total = 0.0f;
        for (uint32_t w = 0; w < warps; ++w) total += red[w * m + row];
        const float r_inv = rsqrtf(total * (1.0f / static_cast<float>(k)) + eps);
        float wv[8];
        if (item == threadIdx.x) {
#pragma unroll
          for (int e = 0; e < 8; ++e) wv[e] = wv0[e];
        } else {
          const float4 w0 = __ldg(reinterpret_cast<const float4*>(weight + (lg << 5) + (q << 3)));
          const float4 w1 = __ldg(reinterpret_cast<const float4*>(weight + (lg << 5) + (q << 3) + 4));
          wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w;
          wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[b][e] = __fmul_rn(__fmul_rn(v[b][e], r_inv), wv[e]);
      }
      stage_octet<kHasLo, kCorrStride, true>(v[b], valid, q, row, lg, xs, xs_stride, corr, 0u, nullptr);
    }
  }
}


// Shared loads that leave the destination untouched where the predicate is false: the
// registers of lanes whose MMA column holds no activation row stay zero for the whole
// kernel, at no per-iteration cost.
__device__ __forceinline__ void lds_v4_if(uint4& v, uint32_t addr, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
               : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
               : "r"(addr), "r"(static_cast<uint32_t>(pred)));
}
__device__ __forceinline__ void lds_f32_if(float& v, uint32_t addr, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p ld.shared.f32 %0, [%1];\n\t}"
               : "+f"(v)
               : "r"(addr), "r"(static_cast<uint32_t>(pred)));
}

// {corr, 2^-e} pair of a (group, activation row), see stage_x
__device__ __forceinline__ void lds_v2f_if(float& a, float& b, uint32_t addr, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\t@p ld.shared.v2.f32 {%0,%1}, [%2];\n\t}"
               : "+f"(a), "+f"(b)
               : "r"(addr), "r"(static_cast<uint32_t>(pred)));
}

// D = A.B + C with C read from registers that are not overwritten.
__device__ __forceinline__ void mma_f16_init(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                             float c0, float c1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%10,%11};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c0), "f"(c1));
}

// D = A.B with a zero accumulator.
__device__ __forceinline__ void mma_f16_zero(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

// One CTA per activation row: the row's largest magnitude, then scale[row] = 2^e and
// inv[row] = 2^-e (pow2_prescale).  Kernels that pre-scale whole activation rows (instead of
// 32-k groups) run this first.
template <typename XT>
__global__ void __launch_bounds__(256)
row_scale_kernel(const XT* __restrict__ x, uint32_t k, float* scale, float* inv) {
  const XT* row = x + static_cast<size_t>(blockIdx.x) * k;
  float amax = 0.0f;
  for (uint32_t i = threadIdx.x * 8; i < k; i += blockDim.x * 8) {  // k is a multiple of 64
    float v[8];
    load_x8<XT>(row + i, v);
    amax = fmaxf(amax, absmax8(v));
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  __shared__ float part[8];
  if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, part[w]);
    const Pow2 ps = pow2_prescale(amax);
    scale[blockIdx.x] = ps.scale;
    inv[blockIdx.x] = ps.inv;
  }
}


}  // namespace kq
