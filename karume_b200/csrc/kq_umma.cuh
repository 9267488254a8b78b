// Helpers shared by the tcgen05 GEMM kernels (kq_qgemm_i4.cu, kq_qgemm_i4_x32.cu): mbarriers with
// bounded waits, shared-memory matrix descriptors for the K-major 128-byte-swizzled layout, the
// kind::f16 MMA with bf16 operands, and the swizzled tile addressing.
#pragma once
#include <cuda_bf16.h>

#include <cstdint>

namespace kq {
namespace umma {

constexpr uint32_t kWaitLimit = 1u << 24;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}

// Bounded wait.  Returns false (at once, if another thread already gave up) when the
// barrier did not flip in time; the caller keeps going without blocking.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                             int code) {
  for (uint32_t spins = 0; spins < kWaitLimit; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  *reinterpret_cast<volatile int*>(status) = code;
  return false;
}

// K-major, 128-byte swizzle: rows are 128 B, groups of 8 rows are 1024 B apart (SBO),
// descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(1) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) |
         (static_cast<uint64_t>(2) << 61);
}

// kind::f16 instruction descriptor: f32 accumulate, bf16 A and B, both K-major, M x N.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t mma_m, uint32_t mma_n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((mma_n >> 3) << 17) | ((mma_m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- CTA pairs (cta_group::2): one MMA spans the two CTAs of a cluster -------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// wait_bounded for a barrier that threads of the peer CTA arrive on
__device__ __forceinline__ bool wait_bounded_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                     int code) {
  for (uint32_t spins = 0; spins < kWaitLimit; ++spins) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((spins & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  *reinterpret_cast<volatile int*>(status) = code;
  return false;
}
// M 256 (128 rows per CTA) x N: A and D are each CTA's own rows, B is read half from each CTA.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `cluster_bar` (a shared::cluster address: this CTA's barrier, or the peer's through
// map_to_cta) once the pair's MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

// 8 nibbles of one 32-bit word -> 8 bf16 (16 bytes, k ascending), each
// RNE_bf16(fround((u - 8) * s)).  (word & (0xF << 4e)) | 0x4B000000 is the float
// 2^23 + u * 16^e exactly; subtracting 2^23 + 8 * 16^e leaves (u - 8) * 16^e exactly, and
// the power of sixteen is taken out of the scale (exact), so the one rounding of the
// multiply is the reference's.
__device__ __forceinline__ uint4 dequant8_bf16(uint32_t word, float s) {
  const float s1 = s * 0.0625f, s2 = s * 0.00390625f, s3 = s * 0.000244140625f;
  const uint32_t hi = word >> 16;
  float v[8];
  v[0] = (__uint_as_float((word & 0x000Fu) | 0x4B000000u) - 8388616.0f) * s;
  v[1] = (__uint_as_float((word & 0x00F0u) | 0x4B000000u) - 8388736.0f) * s1;
  v[2] = (__uint_as_float((word & 0x0F00u) | 0x4B000000u) - 8390656.0f) * s2;
  v[3] = (__uint_as_float((word & 0xF000u) | 0x4B000000u) - 8421376.0f) * s3;
  v[4] = (__uint_as_float((hi & 0x000Fu) | 0x4B000000u) - 8388616.0f) * s;
  v[5] = (__uint_as_float((hi & 0x00F0u) | 0x4B000000u) - 8388736.0f) * s1;
  v[6] = (__uint_as_float((hi & 0x0F00u) | 0x4B000000u) - 8390656.0f) * s2;
  v[7] = (__uint_as_float((hi & 0xF000u) | 0x4B000000u) - 8421376.0f) * s3;
  uint4 out;
  __nv_bfloat162 p;
  p = __floats2bfloat162_rn(v[0], v[1]); out.x = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(v[2], v[3]); out.y = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(v[4], v[5]); out.z = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(v[6], v[7]); out.w = *reinterpret_cast<uint32_t*>(&p);
  return out;
}

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// byte offset of 16-byte piece c (0..7) of tile row r in the swizzled K-major layout
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

}  // namespace umma
}  // namespace kq
