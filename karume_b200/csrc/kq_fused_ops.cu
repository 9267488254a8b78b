// The matmul's neighbours in a decoder layer as kernels of their own: rms_norm, the SiLU gate
// (silu(gate) * up) and the residual add.  kq_linear_fused runs them around a linear when the
// call is not being recorded into a fused plan (inside a plan the persistent kernel does the
// same arithmetic in its activation staging and its epilogue, kq_plan.cu); they are also
// exported as ops of their own.
//
//   rms_norm  out[r, i] = x[r, i] * rsqrt(mean_r(x^2) + eps) * weight[i]
//             (packages/runtime/src/kernels/rms-norm.ts:1-25, :60-90: one block per row, sum of
//             squares in one pass, the mean is not subtracted, eps inside the root, the
//             products evaluated left to right in f32)
//   silu_mul  out[i] = (gate[i] * sigmoid(gate[i])) * up[i], sigmoid in the reference's stable
//             form t = exp(-|x|), x < 0 ? t / (1 + t) : 1 / (1 + t)
//             (packages/runtime/src/codegen/elementwise.ts:187-190; the SiLU pair is the fusion
//             rule of packages/runtime/src/runtime/fusion.ts:453-511, kernel
//             packages/runtime/src/kernels/silu.ts), every product rounded to f32
//   add       out[i] = a[i] + b[i]
#include "kq_common.cuh"
#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kNormThreads = 256;

__global__ void __launch_bounds__(kNormThreads)
rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ weight, float* __restrict__ out, uint32_t rows,
                uint32_t dim, float eps) {
  __shared__ float part[kNormThreads / 32];
  __shared__ float inv_s;
  for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + static_cast<size_t>(row) * dim;
    float acc = 0.0f;
    for (uint32_t i = threadIdx.x; i < dim; i += kNormThreads) acc = fmaf(xr[i], xr[i], acc);
    acc = warp_sum(acc);
    if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.0f;
      for (int w = 0; w < kNormThreads / 32; ++w) total += part[w];  // fixed order
      inv_s = rsqrtf(total * (1.0f / static_cast<float>(dim)) + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    float* orow = out + static_cast<size_t>(row) * dim;
    for (uint32_t i = threadIdx.x; i < dim; i += kNormThreads) orow[i] = __fmul_rn(__fmul_rn(xr[i], inv), weight[i]);
    __syncthreads();  // part / inv_s are rewritten by the next row
  }
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ out, uint64_t count) {
  for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < count; i += static_cast<uint64_t>(gridDim.x) * 256ull)
    out[i] = silu_mul(gate[i], up[i]);
}

__global__ void __launch_bounds__(256)
add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, uint64_t count) {
  for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < count; i += static_cast<uint64_t>(gridDim.x) * 256ull)
    out[i] = __fadd_rn(a[i], b[i]);
}

int grid_for(uint64_t count, int sm_count) {
  const uint64_t blocks = (count + 255) / 256;
  const uint64_t cap = static_cast<uint64_t>(sm_count) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

cudaError_t launch_rms_norm(const LaunchEnv& env, const float* x, const float* weight, float eps, float* out,
                            uint32_t rows, uint32_t dim) {
  const int grid = static_cast<int>(rows < static_cast<uint32_t>(env.sm_count) * 4u ? rows : env.sm_count * 4);
  rms_norm_kernel<<<grid, kNormThreads, 0, env.stream>>>(x, weight, out, rows, dim, eps);
  return cudaGetLastError();
}

cudaError_t launch_silu_mul(const LaunchEnv& env, const float* gate, const float* up, float* out, uint64_t count) {
  silu_mul_kernel<<<grid_for(count, env.sm_count), 256, 0, env.stream>>>(gate, up, out, count);
  return cudaGetLastError();
}

cudaError_t launch_add(const LaunchEnv& env, const float* a, const float* b, float* out, uint64_t count) {
  add_kernel<<<grid_for(count, env.sm_count), 256, 0, env.stream>>>(a, b, out, count);
  return cudaGetLastError();
}

}  // namespace kq
