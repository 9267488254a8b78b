// Device-side helpers shared by every kernel of libkq: the dequant rules, exact
// widening loads of the activation dtypes and the addressing of the tiled int4
// layout.  Keeping the dequant rule in ONE place is deliberate: the GEMV, the
// tensor-core GEMM's tile fill and the f32 expansion all call the functions below,
// so a weight cannot decode differently depending on which kernel reads it.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace kq {

// ---- dequant rules ---------------------------------------------------------
// int4: value = fround(f32(u - 8) * scale) — exactly one f32 rounding
// (packages/runtime/src/kernels/weight-storage.ts:159-187,
//  packages/runtime/src/format/i4.ts:113).  __fmul_rn keeps the product a separate,
// correctly rounded multiply: it can neither be contracted into a following FMA nor
// reassociated with the activation.
__device__ __forceinline__ float dequant_i4(uint32_t nibble, float scale) {
  return __fmul_rn(static_cast<float>(static_cast<int>(nibble) - 8), scale);
}

// int8: value = fround(f32(q) * scale)
// (packages/runtime/src/kernels/weight-storage.ts:191-209,
//  packages/runtime/src/format/i8.ts:107).
__device__ __forceinline__ float dequant_i8(int q, float scale) {
  return __fmul_rn(static_cast<float>(q), scale);
}

// Companion scale -> f32.  binary16 widens exactly, subnormals included
// (packages/runtime/src/format/f16.ts:23-36); the build never enables flush-to-zero.
template <bool kF16>
__device__ __forceinline__ float load_scale(const void* base, size_t index) {
  if constexpr (kF16) {
    return __half2float(reinterpret_cast<const __half*>(base)[index]);
  } else {
    return reinterpret_cast<const float*>(base)[index];
  }
}

// ---- activation loads (exact widening to f32) --------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// ---- tiled int4 layout (group size 32) -----------------------------------------
// A weight [n, k] with n % 16 == 0 and k % 64 == 0 is stored as chunks.  Chunk
// (R, J) holds rows 16R..16R+15 and the two scale groups 2J, 2J+1 (64 k-values):
//
//   bytes [0, 512)   : 32 lanes x 16 B.  Lane L = 4*g + t (g = 0..7, t = 0..3) holds
//                      four 32-bit words copied verbatim from the row-major payload:
//                        word 0 = row 16R+g  , group 2J  , bytes 4t..4t+3 of the group
//                        word 1 = row 16R+g+8, group 2J  , same bytes
//                        word 2 = row 16R+g  , group 2J+1, same bytes
//                        word 3 = row 16R+g+8, group 2J+1, same bytes
//                      (a group's 32 nibbles are 16 bytes; byte b of a group holds
//                      elements 2b (low nibble) and 2b+1 (high nibble) of that group).
//   bytes [512, 512+8*4*S) : scales, S = sizeof(scale element); entry g holds
//                      { s[16R+g][2J], s[16R+g+8][2J], s[16R+g][2J+1], s[16R+g+8][2J+1] }.
//
// Chunks of one 16-row block are contiguous in J, so a warp streaming a row block
// reads one linear byte range; the layout is a permutation of payload + scale bytes
// (nothing is padded or expanded).
constexpr uint32_t kTileRows = 16;
constexpr uint32_t kChunkK = 64;
constexpr uint32_t kChunkWeightBytes = 512;

__host__ __device__ __forceinline__ uint32_t chunk_bytes(uint32_t scale_elem_bytes) {
  return kChunkWeightBytes + 8u * 4u * scale_elem_bytes;
}

struct TiledPos {
  size_t word_offset;   // byte offset of the 32-bit word holding the element
  uint32_t nibble;      // 0..7 position inside that word
  size_t scale_offset;  // byte offset of the element's group scale
};

__host__ __device__ __forceinline__ TiledPos tiled_i4_locate(uint32_t row, uint32_t kk, uint32_t k,
                                                            uint32_t scale_elem_bytes) {
  const uint32_t R = row / kTileRows, rr = row % kTileRows;
  const uint32_t g = rr & 7u, upper = rr >> 3;
  const uint32_t group = kk >> 5, J = group >> 1, jj = group & 1u;
  const uint32_t in_group = kk & 31u, t = in_group >> 3, e = in_group & 7u;
  const size_t base = (static_cast<size_t>(R) * (k / kChunkK) + J) * chunk_bytes(scale_elem_bytes);
  TiledPos pos;
  pos.word_offset = base + (4u * g + t) * 16u + (jj * 2u + upper) * 4u;
  pos.nibble = e;
  pos.scale_offset = base + kChunkWeightBytes + (g * 4u + jj * 2u + upper) * scale_elem_bytes;
  return pos;
}

// ---- tiled int8 layout -------------------------------------------------------------
// A weight [n, k] with n % 16 == 0 and k % 32 == 0 is stored as 512-byte chunks; chunk
// (R, J) holds rows 16R..16R+15 and k 32J..32J+31.  Lane L = 4*g + t owns 16 B = four
// 32-bit words, each four consecutive weights of one row with the sign bit flipped
// (byte = q + 128, an unsigned value 0..255):
//   word 0 = row 16R+g  , k 32J    + 4t .. +3        word 1 = row 16R+g+8, same k
//   word 2 = row 16R+g  , k 32J+16 + 4t .. +3        word 3 = row 16R+g+8, same k
// The per-output-channel scales stay a plain [n] array next to it.
constexpr uint32_t kChunkK8 = 32;

__host__ __device__ __forceinline__ size_t tiled_i8_locate(uint32_t row, uint32_t kk, uint32_t k) {
  const uint32_t R = row / kTileRows, rr = row % kTileRows;
  const uint32_t g = rr & 7u, upper = rr >> 3;
  const uint32_t J = kk >> 5, in = kk & 31u, half = in >> 4, q = in & 15u, t = q >> 2, b = q & 3u;
  return (static_cast<size_t>(R) * (k / kChunkK8) + J) * 512u + (4u * g + t) * 16u + (half * 2u + upper) * 4u + b;
}

// ---- SiLU gate -------------------------------------------------------------------
// sigmoid in the reference's stable form (packages/runtime/src/codegen/elementwise.ts:187-190)
// and silu(gate) * up with every product rounded to f32, as the reference's sigmoid -> mul -> mul
// node sequence rounds them (packages/runtime/src/kernels/silu.ts).
__device__ __forceinline__ float sigmoid_stable(float x) {
  const float t = expf(-fabsf(x));
  return x < 0.0f ? __fdiv_rn(t, __fadd_rn(1.0f, t)) : __fdiv_rn(1.0f, __fadd_rn(1.0f, t));
}
__device__ __forceinline__ float silu_mul(float gate, float up) {
  return __fmul_rn(__fmul_rn(gate, sigmoid_stable(gate)), up);
}

// ---- misc ----------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

// Programmatic dependent launch: no-ops when the launch carries no such attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_prior_grid() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace kq
