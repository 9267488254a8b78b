// C ABI of libkq (see include/kq.h): context, buffers, weight residency, the linear
// op's shape checks and kernel choice, CUDA-graph plans and timing.  There is no CPU
// path anywhere in this file: a request no kernel covers is an error.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "kq_internal.h"

using kq::Weight;

struct kq_ctx {
  int device = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  bool overlap = true;
  bool capturing = false;
  std::string error;
  std::unordered_map<uint64_t, Weight*> weights;
  std::unordered_map<uint64_t, cudaGraphExec_t> graphs;
  std::unordered_map<uint64_t, uint64_t> graph_kernels;  // kernel nodes per recorded graph
  std::unordered_map<uint64_t, kq::Plan*> plans;
  kq::Plan* recording = nullptr;  // non-null between kq_plan_begin and kq_plan_end
  kq::Comm* comm = nullptr;       // tensor-parallel exchange, if created
  std::string recording_refusal;  // first reason an op could not be fused
  uint64_t capture_mark = 0;
  uint64_t next_handle = 1;
  void* workspace = nullptr;
  uint64_t workspace_bytes = 0;
  unsigned int* counters = nullptr;
  uint32_t counter_count = 0;
  int* gemm_status_host = nullptr;  // mapped, page-locked: non-zero once a bounded wait of a tcgen05 kernel gave up
  int* gemm_status_dev = nullptr;
  // neighbours kq_linear_fused hands to the next wide-GEMV launch (set and cleared around one call)
  const float* nb_norm_weight = nullptr;
  float nb_norm_eps = 0.0f;
  const float* nb_residual = nullptr;
  int sm_count = 0;
  cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
  uint64_t launches = 0;
  void* host_x = nullptr;   // staging for kq_linear_host
  void* host_dev_x = nullptr;
  void* host_dev_out = nullptr;
  uint64_t host_x_bytes = 0, host_out_bytes = 0;
  float* zero_bias = nullptr;  // kq_linear_reduce's unfused path: ranks other than 0 add no bias
  uint64_t zero_bias_count = 0;
  int* idot_sums = nullptr;  // integer sums of the quantised activations (kq_linear_a8)
  uint64_t idot_sums_bytes = 0;
  float* fused_xn = nullptr;  // kq_linear_fused outside a plan: the normalised activations ...
  uint64_t fused_xn_bytes = 0;
  float* fused_gu = nullptr;  // ... and the gate / up outputs in front of the SiLU gate
  uint64_t fused_gu_bytes = 0;
};

namespace {

std::string g_init_error;

int fail(kq_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list args;
  va_start(args, fmt);
  vsnprintf(buf, sizeof buf, fmt, args);
  va_end(args);
  if (ctx) ctx->error = buf;
  else g_init_error = buf;
  return code;
}

int cuda_fail(kq_ctx* ctx, cudaError_t e, const char* what) {
  const int code = e == cudaErrorMemoryAllocation ? KQ_ERR_OOM : KQ_ERR_CUDA;
  return fail(ctx, code, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

#define KQ_CUDA(ctx, call)                                  \
  do {                                                      \
    cudaError_t kq_e_ = (call);                             \
    if (kq_e_ != cudaSuccess) return cuda_fail(ctx, kq_e_, #call); \
  } while (0)

struct DeviceGuard {
  int previous = -1;
  explicit DeviceGuard(int device) {
    cudaGetDevice(&previous);
    if (previous != device) cudaSetDevice(device);
    else previous = -1;
  }
  ~DeviceGuard() {
    if (previous >= 0) cudaSetDevice(previous);
  }
};

kq::LaunchEnv env_of(kq_ctx* ctx) {
  kq::LaunchEnv env;
  env.stream = ctx->stream;
  env.overlap = ctx->overlap;
  env.workspace = ctx->workspace;
  env.workspace_bytes = ctx->workspace_bytes;
  env.counters = ctx->counters;
  env.counter_count = ctx->counter_count;
  env.sm_count = ctx->sm_count;
  env.status = ctx->gemm_status_dev;
  env.norm_weight = ctx->nb_norm_weight;
  env.norm_eps = ctx->nb_norm_eps;
  env.residual = ctx->nb_residual;
  return env;
}

bool is_pow2(uint32_t v) { return v && !(v & (v - 1)); }

Weight* find_weight(kq_ctx* ctx, kq_weight h) {
  auto it = ctx->weights.find(h);
  return it == ctx->weights.end() ? nullptr : it->second;
}

uint32_t dtype_bytes(int dtype) { return dtype == KQ_F32 ? 4u : 2u; }

// Storage-contract checks shared by the upload entry points.
int check_storage(kq_ctx* ctx, int storage, uint64_t payload_bytes, uint64_t scale_bytes,
                  int scale_dtype, uint32_t n, uint32_t k, uint32_t group_size) {
  if (scale_dtype != KQ_F32 && scale_dtype != KQ_F16)
    return fail(ctx, KQ_ERR_BAD_ARG, "scale_dtype %d: companion scales are F32 or F16", scale_dtype);
  const uint64_t numel = static_cast<uint64_t>(n) * k;
  const uint64_t sb = dtype_bytes(scale_dtype);
  if (storage == KQ_STORAGE_I4) {
    // packages/runtime/src/kernels/weight-storage.ts:56-70: power of two, >= 16
    if (!is_pow2(group_size) || group_size < 16)
      return fail(ctx, KQ_ERR_SHAPE, "i4 group_size %u is not a power of two >= 16", group_size);
    // packages/runtime/src/format/i4.ts:79-82
    if (k % group_size != 0)
      return fail(ctx, KQ_ERR_SHAPE, "group_size %u does not divide the row length %u", group_size, k);
    // packages/runtime/src/format/i4.ts:71-77
    if (payload_bytes * 2 != numel)
      return fail(ctx, KQ_ERR_SHAPE, "i4 payload of %llu bytes does not match shape [%u,%u] (%llu needed)",
                  (unsigned long long)payload_bytes, n, k, (unsigned long long)(numel / 2));
    // packages/runtime/src/format/i4.ts:84-100: group form [n, k/group_size]
    if (scale_bytes != static_cast<uint64_t>(n) * (k / group_size) * sb)
      return fail(ctx, KQ_ERR_SHAPE, "i4 scale of %llu bytes is not the group form [%u,%u]",
                  (unsigned long long)scale_bytes, n, k / group_size);
  } else if (storage == KQ_STORAGE_I8) {
    // docs/ir-v1.md:151-155: group quantisation exists for i4 only
    if (group_size != 0)
      return fail(ctx, KQ_ERR_SHAPE, "group_size %u on i8 storage: group quantisation is i4-only", group_size);
    // packages/runtime/src/format/i8.ts:86-91
    if (payload_bytes != numel)
      return fail(ctx, KQ_ERR_SHAPE, "i8 payload of %llu bytes does not match shape [%u,%u]",
                  (unsigned long long)payload_bytes, n, k);
    if (scale_bytes != static_cast<uint64_t>(n) * sb)
      return fail(ctx, KQ_ERR_SHAPE, "i8 scale of %llu bytes is not the per-output-channel form [%u,1]",
                  (unsigned long long)scale_bytes, n);
  } else {
    return fail(ctx, KQ_ERR_BAD_ARG, "storage %d: expected KQ_STORAGE_I4 or KQ_STORAGE_I8", storage);
  }
  return KQ_OK;
}

int upload_checked(kq_ctx* ctx, int storage, const void* payload, uint64_t payload_bytes,
                   const void* scale, uint64_t scale_bytes, int scale_dtype, uint32_t n, uint32_t k,
                   uint32_t group_size, kq_weight* out) {
  DeviceGuard guard(ctx->device);
  if (ctx->capturing) return fail(ctx, KQ_ERR_STATE, "kq_weight_upload during graph capture");
  Weight* w = new Weight();
  w->storage = storage;
  w->scale_dtype = scale_dtype;
  w->n = n;
  w->k = k;
  w->group_size = group_size;
  w->payload_bytes = payload_bytes;
  w->scale_bytes = scale_bytes;
  void* d_payload = nullptr;
  void* d_scale = nullptr;
  auto cleanup = [&]() {
    if (d_payload) cudaFree(d_payload);
    if (d_scale) cudaFree(d_scale);
    delete w;
  };
  // i8 payloads are padded to a 4-byte multiple like the reference's GPU buffer
  // (packages/runtime/src/format/i8.ts:34-40); the pad is never read.
  const uint64_t padded = (payload_bytes + 15) & ~uint64_t(15);
  cudaError_t e = cudaMalloc(&d_payload, padded ? padded : 16);
  if (e == cudaSuccess) e = cudaMalloc(&d_scale, scale_bytes ? scale_bytes : 16);
  if (e == cudaSuccess && padded) e = cudaMemsetAsync(d_payload, 0, padded, ctx->stream);
  if (e == cudaSuccess && payload_bytes)
    e = cudaMemcpyAsync(d_payload, payload, payload_bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess && scale_bytes)
    e = cudaMemcpyAsync(d_scale, scale, scale_bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (e != cudaSuccess) {
    cleanup();
    return cuda_fail(ctx, e, "weight upload");
  }
  if (kq::tiled_i4_eligible(storage, n, k, group_size)) {
    void* tiled = nullptr;
    e = cudaMalloc(&tiled, payload_bytes + scale_bytes);
    if (e == cudaSuccess)
      e = kq::launch_repack_i4(ctx->stream, static_cast<const uint8_t*>(d_payload), d_scale, scale_dtype,
                               n, k, static_cast<uint8_t*>(tiled));
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
      if (tiled) cudaFree(tiled);
      cleanup();
      return cuda_fail(ctx, e, "weight repack");
    }
    ctx->launches += 1;
    cudaFree(d_payload);
    cudaFree(d_scale);
    w->layout = kq::kLayoutTiledI4;
    w->data = tiled;
    w->scale = nullptr;
  } else if (kq::tiled_i8_eligible(storage, n, k)) {
    void* tiled = nullptr;
    e = cudaMalloc(&tiled, payload_bytes);
    if (e == cudaSuccess)
      e = kq::launch_repack_i8(ctx->stream, static_cast<const uint8_t*>(d_payload), n, k, static_cast<uint8_t*>(tiled));
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
      if (tiled) cudaFree(tiled);
      cleanup();
      return cuda_fail(ctx, e, "weight repack");
    }
    ctx->launches += 1;
    cudaFree(d_payload);
    w->layout = kq::kLayoutTiledI8;
    w->data = tiled;
    w->scale = d_scale;
  } else {
    e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
      cleanup();
      return cuda_fail(ctx, e, "weight upload");
    }
    w->layout = kq::kLayoutNative;
    w->data = d_payload;
    w->scale = d_scale;
  }
  const uint64_t handle = ctx->next_handle++;
  ctx->weights[handle] = w;
  *out = handle;
  return KQ_OK;
}

int check_linear_args(kq_ctx* ctx, const Weight* w, uint64_t x, int x_dtype, uint64_t bias, uint64_t out) {
  if (!w) return fail(ctx, KQ_ERR_BAD_ARG, "unknown weight handle");
  if (x_dtype != KQ_F32 && x_dtype != KQ_F16 && x_dtype != KQ_BF16)
    return fail(ctx, KQ_ERR_BAD_ARG, "x_dtype %d: expected KQ_F32, KQ_F16 or KQ_BF16", x_dtype);
  if (!x || !bias || !out)
    return fail(ctx, KQ_ERR_BAD_ARG, "x, bias and out must be device pointers (bias is not optional: linear has arity 3)");
  if ((x & 15u) || (out & 3u) || (bias & 3u))
    return fail(ctx, KQ_ERR_BAD_ARG, "x must be 16-byte aligned, bias and out 4-byte aligned");
  return KQ_OK;
}

int run_linear(kq_ctx* ctx, uint32_t count, const kq_weight* handles, uint64_t x, int x_dtype,
               const uint64_t* bias, const uint64_t* out, uint32_t m, const kq::LinearFusion* fusion = nullptr) {
  if (count < 1 || count > (uint32_t)kq::kMaxMulti)
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_multi: count %u outside 1..%d", count, kq::kMaxMulti);
  kq::LinearTarget targets[kq::kMaxMulti];
  for (uint32_t i = 0; i < count; ++i) {
    const Weight* w = find_weight(ctx, handles[i]);
    const int rc = check_linear_args(ctx, w, x, x_dtype, bias[i], out[i]);
    if (rc != KQ_OK) return rc;
    if (w->k != find_weight(ctx, handles[0])->k)
      return fail(ctx, KQ_ERR_SHAPE, "kq_linear_multi: weight %u has k=%u, weight 0 has k=%u", i, w->k,
                  find_weight(ctx, handles[0])->k);
    targets[i] = kq::LinearTarget{w, reinterpret_cast<const float*>(bias[i]), reinterpret_cast<float*>(out[i])};
  }
  if (ctx->recording) {
    const char* why = kq::plan_add_linear(ctx->recording, static_cast<int>(count), targets,
                                          reinterpret_cast<const void*>(x), x_dtype, m,
                                          fusion ? *fusion : kq::LinearFusion{});
    if (why[0] != 0 && ctx->recording_refusal.empty()) ctx->recording_refusal = why;
    return KQ_OK;
  }
  if (m == 0) return KQ_OK;
  DeviceGuard guard(ctx->device);
  const kq::LaunchEnv env = env_of(ctx);
  const uint32_t xb = dtype_bytes(x_dtype);
  bool all_tiled = true, same_scale = true;
  for (uint32_t i = 0; i < count; ++i) {
    all_tiled = all_tiled && targets[i].w->layout == kq::kLayoutTiledI4;
    same_scale = same_scale && targets[i].w->scale_dtype == targets[0].w->scale_dtype;
  }
  if (all_tiled && kq::qgemm_i4_supports(*targets[0].w, x_dtype, m)) {
    // Prefill: bf16 activations, more than 16 rows -> tcgen05 GEMM, one launch per weight.
    for (uint32_t i = 0; i < count; ++i) {
      if (targets[i].w->n == 0) continue;
      int extra = 0;
      cudaError_t e = kq::launch_qgemm_i4(env, targets[i], reinterpret_cast<const void*>(x), m, ctx->gemm_status_dev, &extra);
      if (e != cudaSuccess) return cuda_fail(ctx, e, "qgemm_i4 launch");
      ctx->launches += 1 + extra;
    }
    return KQ_OK;
  }
  bool x32 = all_tiled;
  for (uint32_t i = 0; i < count && x32; ++i)
    x32 = targets[i].w->n == 0 || kq::qgemm_i4_x32_supports(*targets[i].w, x_dtype, m, ctx->workspace ? ctx->workspace_bytes : 0);
  if (x32) {
    // Prefill with f32 / binary16 activations: the split-operand tcgen05 GEMM, one weight at a time.
    for (uint32_t i = 0; i < count; ++i) {
      if (targets[i].w->n == 0) continue;
      int launched = 0;
      cudaError_t e = kq::launch_qgemm_i4_x32(env, targets[i], reinterpret_cast<const void*>(x), x_dtype, m, ctx->gemm_status_dev,
                                              &launched);
      if (e != cudaSuccess) return cuda_fail(ctx, e, "qgemm_i4_x32 launch");
      ctx->launches += launched;
    }
    return KQ_OK;
  }
  if (all_tiled && same_scale) {
    // Tiled int4: row panels of at most 16 activation rows per launch.
    for (uint32_t m0 = 0; m0 < m; m0 += 16) {
      const uint32_t mm = std::min<uint32_t>(16u, m - m0);
      kq::LinearTarget panel[kq::kMaxMulti];
      for (uint32_t i = 0; i < count; ++i)
        panel[i] = kq::LinearTarget{targets[i].w, targets[i].bias,
                                    targets[i].out + static_cast<size_t>(m0) * targets[i].w->n};
      int launched = 0;
      const void* xp = reinterpret_cast<const uint8_t*>(x) + static_cast<size_t>(m0) * targets[0].w->k * xb;
      cudaError_t e = kq::launch_qgemv_i4(env, static_cast<int>(count), panel, xp, x_dtype, mm, &launched);
      if (e != cudaSuccess) return cuda_fail(ctx, e, "qgemv_i4 launch");
      ctx->launches += launched;
    }
    return KQ_OK;
  }
  // Everything else: one generic launch per weight.
  for (uint32_t i = 0; i < count; ++i) {
    const Weight& w = *targets[i].w;
    if (w.layout == kq::kLayoutTiledI4) {
      kq::LinearTarget one = targets[i];
      for (uint32_t m0 = 0; m0 < m; m0 += 16) {
        const uint32_t mm = std::min<uint32_t>(16u, m - m0);
        kq::LinearTarget panel{one.w, one.bias, one.out + static_cast<size_t>(m0) * w.n};
        int launched = 0;
        const void* xp = reinterpret_cast<const uint8_t*>(x) + static_cast<size_t>(m0) * w.k * xb;
        cudaError_t e = kq::launch_qgemv_i4(env, 1, &panel, xp, x_dtype, mm, &launched);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qgemv_i4 launch");
        ctx->launches += launched;
      }
      continue;
    }
    if (w.n == 0) continue;
    if (kq::qgemm_i8_supports(w, x_dtype, m)) {
      // Prefill over an int8 weight: the tcgen05 GEMM with the int8 producer path.
      int extra = 0;
      cudaError_t e = kq::launch_qgemm_i4(env, targets[i], reinterpret_cast<const void*>(x), m, ctx->gemm_status_dev, &extra);
      if (e != cudaSuccess) return cuda_fail(ctx, e, "qgemm_i8 launch");
      ctx->launches += 1 + extra;
      continue;
    }
    if (w.layout == kq::kLayoutTiledI8) {
      // Tiled int8: row panels of at most 16 activation rows per launch.
      for (uint32_t m0 = 0; m0 < m; m0 += 16) {
        const uint32_t mm = std::min<uint32_t>(16u, m - m0);
        kq::LinearTarget panel{targets[i].w, targets[i].bias, targets[i].out + static_cast<size_t>(m0) * w.n};
        const void* xp = reinterpret_cast<const uint8_t*>(x) + static_cast<size_t>(m0) * w.k * xb;
        cudaError_t e8 = kq::launch_qgemv_i8(env, panel, xp, x_dtype, mm);
        if (e8 != cudaSuccess) return cuda_fail(ctx, e8, "qgemv_i8 launch");
        ctx->launches += 1;
      }
      continue;
    }
    cudaError_t e = kq::launch_linear_generic(env, w, reinterpret_cast<const void*>(x), x_dtype,
                                              targets[i].bias, targets[i].out, m);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "generic linear launch");
    ctx->launches += 1;
  }
  return KQ_OK;
}

}  // namespace

namespace kq {
void set_global_error(const std::string& message) { g_init_error = message; }
int ctx_fail(kq_ctx* ctx, int code, const std::string& message) { return fail(ctx, code, "%s", message.c_str()); }
}  // namespace kq

extern "C" {

const char* kq_version(void) { return "kq 0.1 sm_100a"; }

int kq_init(int device, uint64_t workspace_bytes, kq_ctx** out) {
  if (!out) return fail(nullptr, KQ_ERR_BAD_ARG, "kq_init: out is null");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceCount");
  if (device < 0 || device >= count)
    return fail(nullptr, KQ_ERR_BAD_ARG, "kq_init: device %d outside 0..%d", device, count - 1);
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceProperties");
  if (prop.major != 10)
    return fail(nullptr, KQ_ERR_UNSUPPORTED,
                "kq_init: device %d is sm_%d%d; this library carries sm_100a code only and has no other path",
                device, prop.major, prop.minor);
  DeviceGuard guard(device);
  kq_ctx* ctx = new kq_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->workspace_bytes = workspace_bytes ? workspace_bytes : (256ull << 20);
  ctx->counter_count = 8192;
  e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(&ctx->workspace, ctx->workspace_bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&ctx->counters), ctx->counter_count * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemset(ctx->counters, 0, ctx->counter_count * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&ctx->gemm_status_host), sizeof(int), cudaHostAllocMapped);
  if (e == cudaSuccess) {
    ctx->gemm_status_host[0] = 0;
    e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->gemm_status_dev), ctx->gemm_status_host, 0);
  }
  if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev_start);
  if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev_stop);
  if (e != cudaSuccess) {
    const int rc = cuda_fail(nullptr, e, "kq_init");
    kq_destroy(ctx);
    return rc;
  }
  ctx->stream = ctx->own_stream;
  *out = ctx;
  return KQ_OK;
}

void kq_destroy(kq_ctx* ctx) {
  if (!ctx) return;
  DeviceGuard guard(ctx->device);
  if (ctx->own_stream) cudaStreamSynchronize(ctx->own_stream);
  for (auto& kv : ctx->graphs) cudaGraphExecDestroy(kv.second);
  for (auto& kv : ctx->plans) kq::plan_destroy(kv.second);
  if (ctx->comm) kq::comm_destroy(ctx->comm);
  if (ctx->recording) kq::plan_destroy(ctx->recording);
  for (auto& kv : ctx->weights) {
    if (kv.second->data) cudaFree(kv.second->data);
    if (kv.second->scale) cudaFree(kv.second->scale);
    delete kv.second;
  }
  if (ctx->workspace) cudaFree(ctx->workspace);
  if (ctx->counters) cudaFree(ctx->counters);
  if (ctx->gemm_status_host) cudaFreeHost(ctx->gemm_status_host);
  if (ctx->host_x) cudaFreeHost(ctx->host_x);
  if (ctx->host_dev_x) cudaFree(ctx->host_dev_x);
  if (ctx->host_dev_out) cudaFree(ctx->host_dev_out);
  if (ctx->idot_sums) cudaFree(ctx->idot_sums);
  if (ctx->fused_xn) cudaFree(ctx->fused_xn);
  if (ctx->fused_gu) cudaFree(ctx->fused_gu);
  if (ctx->zero_bias) cudaFree(ctx->zero_bias);
  if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
  if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  delete ctx;
}

const char* kq_last_error(kq_ctx* ctx) { return ctx ? ctx->error.c_str() : g_init_error.c_str(); }

int kq_set_stream(kq_ctx* ctx, uint64_t cuda_stream) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->capturing) return fail(ctx, KQ_ERR_STATE, "kq_set_stream during graph capture");
  ctx->stream = cuda_stream ? reinterpret_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
  return KQ_OK;
}

int kq_set_overlap(kq_ctx* ctx, int enabled) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  ctx->overlap = enabled != 0;
  return KQ_OK;
}

int kq_sync(kq_ctx* ctx) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->capturing || ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_sync while a graph or plan is being recorded");
  DeviceGuard guard(ctx->device);
  KQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (*reinterpret_cast<volatile int*>(ctx->gemm_status_host) != 0) {
    const int code = *reinterpret_cast<volatile int*>(ctx->gemm_status_host);
    *reinterpret_cast<volatile int*>(ctx->gemm_status_host) = 0;
    return fail(ctx, KQ_ERR_TIMEOUT, "a bounded wait inside a tcgen05 kernel gave up (stage %d); its outputs are not valid", code);
  }
  if (ctx->comm && kq::comm_take_status(ctx->comm) != 0)
    return fail(ctx, KQ_ERR_TIMEOUT, "kq_all_reduce: a peer did not arrive within the bounded wait; the outputs are not valid");
  for (auto& kv : ctx->plans) {
    const int st = kq::plan_take_status(kv.second);
    if (st != 0)
      return fail(ctx, KQ_ERR_TIMEOUT, "a bounded wait inside the fused plan kernel gave up (%s); its outputs are not valid",
                  st == 1 ? "grid barrier between ops" : "weight copy completion");
  }
  return KQ_OK;
}

int kq_buffer_alloc(kq_ctx* ctx, uint64_t bytes, uint64_t* out_dptr) {
  if (!ctx || !out_dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_buffer_alloc: null argument");
  DeviceGuard guard(ctx->device);
  void* p = nullptr;
  KQ_CUDA(ctx, cudaMalloc(&p, bytes ? bytes : 16));
  *out_dptr = reinterpret_cast<uint64_t>(p);
  return KQ_OK;
}

int kq_buffer_free(kq_ctx* ctx, uint64_t dptr) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  DeviceGuard guard(ctx->device);
  KQ_CUDA(ctx, cudaFree(reinterpret_cast<void*>(dptr)));
  return KQ_OK;
}

int kq_buffer_write(kq_ctx* ctx, uint64_t dptr, uint64_t offset, const void* host, uint64_t bytes) {
  if (!ctx || !dptr || (!host && bytes)) return fail(ctx, KQ_ERR_BAD_ARG, "kq_buffer_write: null argument");
  DeviceGuard guard(ctx->device);
  if (ctx->recording) {
    if (bytes) {
      const char* why = kq::plan_add_copy(ctx->recording, true, reinterpret_cast<uint8_t*>(dptr) + offset, const_cast<void*>(host), bytes);
      if (why[0] != 0 && ctx->recording_refusal.empty()) ctx->recording_refusal = why;
    }
    return KQ_OK;
  }
  if (bytes)
    KQ_CUDA(ctx, cudaMemcpyAsync(reinterpret_cast<uint8_t*>(dptr) + offset, host, bytes,
                                 cudaMemcpyHostToDevice, ctx->stream));
  return KQ_OK;
}

int kq_buffer_read(kq_ctx* ctx, uint64_t dptr, uint64_t offset, void* host, uint64_t bytes) {
  if (!ctx || !dptr || (!host && bytes)) return fail(ctx, KQ_ERR_BAD_ARG, "kq_buffer_read: null argument");
  DeviceGuard guard(ctx->device);
  if (ctx->recording) {
    if (bytes) {
      const char* why = kq::plan_add_copy(ctx->recording, false, reinterpret_cast<uint8_t*>(dptr) + offset, host, bytes);
      if (why[0] != 0 && ctx->recording_refusal.empty()) ctx->recording_refusal = why;
    }
    return KQ_OK;
  }
  if (bytes)
    KQ_CUDA(ctx, cudaMemcpyAsync(host, reinterpret_cast<const uint8_t*>(dptr) + offset, bytes,
                                 cudaMemcpyDeviceToHost, ctx->stream));
  return KQ_OK;
}

int kq_host_alloc(kq_ctx* ctx, uint64_t bytes, void** out_host) {
  if (!ctx || !out_host) return fail(ctx, KQ_ERR_BAD_ARG, "kq_host_alloc: null argument");
  DeviceGuard guard(ctx->device);
  KQ_CUDA(ctx, cudaHostAlloc(out_host, bytes ? bytes : 16, cudaHostAllocDefault));
  return KQ_OK;
}

int kq_host_free(kq_ctx* ctx, void* host) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  DeviceGuard guard(ctx->device);
  KQ_CUDA(ctx, cudaFreeHost(host));
  return KQ_OK;
}

int kq_weight_upload(kq_ctx* ctx, int storage, const void* payload, uint64_t payload_bytes,
                     const void* scale, uint64_t scale_bytes, int scale_dtype, uint32_t n, uint32_t k,
                     uint32_t group_size, kq_weight* out) {
  if (!ctx || !out || (!payload && payload_bytes) || (!scale && scale_bytes))
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_weight_upload: null argument");
  *out = 0;
  const int rc = check_storage(ctx, storage, payload_bytes, scale_bytes, scale_dtype, n, k, group_size);
  if (rc != KQ_OK) return rc;
  return upload_checked(ctx, storage, payload, payload_bytes, scale, scale_bytes, scale_dtype, n, k,
                        group_size, out);
}

int kq_weight_upload_shard(kq_ctx* ctx, int storage, const void* payload, uint64_t payload_bytes,
                           const void* scale, uint64_t scale_bytes, int scale_dtype, uint32_t n,
                           uint32_t k, uint32_t group_size, int shard, uint32_t rank, uint32_t world,
                           kq_weight* out) {
  if (!ctx || !out || (!payload && payload_bytes) || (!scale && scale_bytes))
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_weight_upload_shard: null argument");
  *out = 0;
  int rc = check_storage(ctx, storage, payload_bytes, scale_bytes, scale_dtype, n, k, group_size);
  if (rc != KQ_OK) return rc;
  if (world == 0 || rank >= world)
    return fail(ctx, KQ_ERR_BAD_ARG, "shard rank %u outside world %u", rank, world);
  if (shard == KQ_SHARD_NONE || world == 1)
    return upload_checked(ctx, storage, payload, payload_bytes, scale, scale_bytes, scale_dtype, n, k,
                          group_size, out);
  const uint64_t sb = dtype_bytes(scale_dtype);
  const uint8_t* pay = static_cast<const uint8_t*>(payload);
  const uint8_t* scl = static_cast<const uint8_t*>(scale);
  if (shard == KQ_SHARD_COLUMN) {
    if (n % world != 0) return fail(ctx, KQ_ERR_SHAPE, "column shard: n=%u not divisible by world=%u", n, world);
    const uint32_t ns = n / world;
    const uint64_t row_bytes = storage == KQ_STORAGE_I4 ? k / 2 : k;
    const uint64_t scale_row = storage == KQ_STORAGE_I4 ? (k / group_size) * sb : sb;
    if (storage == KQ_STORAGE_I4 && (static_cast<uint64_t>(ns) * k) % 2 != 0)
      return fail(ctx, KQ_ERR_SHAPE, "column shard splits a byte");
    return upload_checked(ctx, storage, pay + static_cast<uint64_t>(rank) * ns * row_bytes, ns * row_bytes,
                          scl + static_cast<uint64_t>(rank) * ns * scale_row, ns * scale_row, scale_dtype,
                          ns, k, group_size, out);
  }
  if (shard == KQ_SHARD_ROW) {
    if (k % world != 0) return fail(ctx, KQ_ERR_SHAPE, "row shard: k=%u not divisible by world=%u", k, world);
    const uint32_t ks = k / world;
    const uint32_t align = storage == KQ_STORAGE_I4 ? group_size : 1;
    if (ks % align != 0)
      return fail(ctx, KQ_ERR_SHAPE, "row shard: k/world=%u is not a multiple of the group size %u", ks, group_size);
    const uint64_t row_bytes = storage == KQ_STORAGE_I4 ? k / 2 : k;
    const uint64_t shard_row = storage == KQ_STORAGE_I4 ? ks / 2 : ks;
    std::vector<uint8_t> cut(static_cast<size_t>(n) * shard_row);
    for (uint32_t r = 0; r < n; ++r)
      memcpy(cut.data() + static_cast<size_t>(r) * shard_row, pay + r * row_bytes + rank * shard_row, shard_row);
    if (storage == KQ_STORAGE_I8) {
      return upload_checked(ctx, storage, cut.data(), cut.size(), scale, scale_bytes, scale_dtype, n, ks, 0, out);
    }
    const uint64_t full_groups = k / group_size, shard_groups = ks / group_size;
    std::vector<uint8_t> scut(static_cast<size_t>(n) * shard_groups * sb);
    for (uint32_t r = 0; r < n; ++r)
      memcpy(scut.data() + static_cast<size_t>(r) * shard_groups * sb,
             scl + (r * full_groups + static_cast<uint64_t>(rank) * shard_groups) * sb, shard_groups * sb);
    return upload_checked(ctx, storage, cut.data(), cut.size(), scut.data(), scut.size(), scale_dtype, n, ks,
                          group_size, out);
  }
  return fail(ctx, KQ_ERR_BAD_ARG, "shard mode %d unknown", shard);
}

int kq_weight_free(kq_ctx* ctx, kq_weight h) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  Weight* w = find_weight(ctx, h);
  if (!w) return fail(ctx, KQ_ERR_BAD_ARG, "kq_weight_free: unknown weight handle");
  DeviceGuard guard(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (w->data) cudaFree(w->data);
  if (w->scale) cudaFree(w->scale);
  delete w;
  ctx->weights.erase(h);
  return KQ_OK;
}

uint64_t kq_weight_resident_bytes(kq_ctx* ctx, kq_weight h) {
  Weight* w = ctx ? find_weight(ctx, h) : nullptr;
  return w ? w->payload_bytes + w->scale_bytes : 0;
}

int kq_weight_shape(kq_ctx* ctx, kq_weight h, uint32_t* out_n, uint32_t* out_k) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  Weight* w = find_weight(ctx, h);
  if (!w || !out_n || !out_k) return fail(ctx, KQ_ERR_BAD_ARG, "kq_weight_shape: bad argument");
  *out_n = w->n;
  *out_k = w->k;
  return KQ_OK;
}

int kq_weight_dequant(kq_ctx* ctx, kq_weight h, uint64_t out_f32_dptr) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  Weight* w = find_weight(ctx, h);
  if (!w || !out_f32_dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_weight_dequant: bad argument");
  DeviceGuard guard(ctx->device);
  cudaError_t e = kq::launch_dequant(env_of(ctx), *w, reinterpret_cast<float*>(out_f32_dptr));
  if (e != cudaSuccess) return cuda_fail(ctx, e, "dequant launch");
  ctx->launches += 1;
  return KQ_OK;
}

int kq_linear(kq_ctx* ctx, kq_weight w, uint64_t x_dptr, int x_dtype, uint64_t bias_dptr,
              uint64_t out_dptr, uint32_t m) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  return run_linear(ctx, 1, &w, x_dptr, x_dtype, &bias_dptr, &out_dptr, m);
}

int kq_linear_multi(kq_ctx* ctx, uint32_t count, const kq_weight* w, uint64_t x_dptr, int x_dtype,
                    const uint64_t* bias_dptr, const uint64_t* out_dptr, uint32_t m) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (!w || !bias_dptr || !out_dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_multi: null argument");
  return run_linear(ctx, count, w, x_dptr, x_dtype, bias_dptr, out_dptr, m);
}

int kq_linear_host(kq_ctx* ctx, kq_weight h, const void* x_host, int x_dtype, uint64_t bias_dptr,
                   float* out_host, uint32_t m) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  Weight* w = find_weight(ctx, h);
  if (!w || !x_host || !out_host) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_host: bad argument");
  if (ctx->capturing || ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_linear_host during a recording");
  if (x_dtype != KQ_F32 && x_dtype != KQ_F16 && x_dtype != KQ_BF16)
    return fail(ctx, KQ_ERR_BAD_ARG, "x_dtype %d unknown", x_dtype);
  DeviceGuard guard(ctx->device);
  const uint64_t xbytes = static_cast<uint64_t>(m) * w->k * dtype_bytes(x_dtype);
  const uint64_t obytes = static_cast<uint64_t>(m) * w->n * sizeof(float);
  if (xbytes > ctx->host_x_bytes) {
    if (ctx->host_dev_x) cudaFree(ctx->host_dev_x);
    ctx->host_dev_x = nullptr;
    ctx->host_x_bytes = 0;
    KQ_CUDA(ctx, cudaMalloc(&ctx->host_dev_x, xbytes));
    ctx->host_x_bytes = xbytes;
  }
  if (obytes > ctx->host_out_bytes) {
    if (ctx->host_dev_out) cudaFree(ctx->host_dev_out);
    ctx->host_dev_out = nullptr;
    ctx->host_out_bytes = 0;
    KQ_CUDA(ctx, cudaMalloc(&ctx->host_dev_out, obytes));
    ctx->host_out_bytes = obytes;
  }
  if (m == 0) return KQ_OK;
  KQ_CUDA(ctx, cudaMemcpyAsync(ctx->host_dev_x, x_host, xbytes, cudaMemcpyHostToDevice, ctx->stream));
  const uint64_t xd = reinterpret_cast<uint64_t>(ctx->host_dev_x);
  const uint64_t od = reinterpret_cast<uint64_t>(ctx->host_dev_out);
  const int rc = run_linear(ctx, 1, &h, xd, x_dtype, &bias_dptr, &od, m);
  if (rc != KQ_OK) return rc;
  KQ_CUDA(ctx, cudaMemcpyAsync(out_host, ctx->host_dev_out, obytes, cudaMemcpyDeviceToHost, ctx->stream));
  return kq_sync(ctx);
}

int kq_graph_begin(kq_ctx* ctx) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->capturing || ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_graph_begin: a recording is already open");
  DeviceGuard guard(ctx->device);
  KQ_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  ctx->capturing = true;
  ctx->capture_mark = ctx->launches;
  return KQ_OK;
}

int kq_graph_end(kq_ctx* ctx, kq_graph* out) {
  if (!ctx || !out) return fail(ctx, KQ_ERR_BAD_ARG, "kq_graph_end: null argument");
  if (!ctx->capturing) return fail(ctx, KQ_ERR_STATE, "kq_graph_end without kq_graph_begin");
  DeviceGuard guard(ctx->device);
  ctx->capturing = false;
  cudaGraph_t graph = nullptr;
  KQ_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &graph));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaGraphInstantiate");
  const uint64_t handle = ctx->next_handle++;
  ctx->graphs[handle] = exec;
  ctx->graph_kernels[handle] = ctx->launches - ctx->capture_mark;
  ctx->launches = ctx->capture_mark;  // recorded, not run
  *out = handle;
  return KQ_OK;
}

int kq_graph_launch(kq_ctx* ctx, kq_graph g) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  auto it = ctx->graphs.find(g);
  if (it == ctx->graphs.end()) return fail(ctx, KQ_ERR_BAD_ARG, "kq_graph_launch: unknown graph handle");
  DeviceGuard guard(ctx->device);
  KQ_CUDA(ctx, cudaGraphLaunch(it->second, ctx->stream));
  ctx->launches += ctx->graph_kernels[g];
  return KQ_OK;
}

int kq_graph_free(kq_ctx* ctx, kq_graph g) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  auto it = ctx->graphs.find(g);
  if (it == ctx->graphs.end()) return fail(ctx, KQ_ERR_BAD_ARG, "kq_graph_free: unknown graph handle");
  DeviceGuard guard(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  cudaGraphExecDestroy(it->second);
  ctx->graphs.erase(it);
  ctx->graph_kernels.erase(g);
  return KQ_OK;
}

int kq_linear_static(kq_ctx* ctx, kq_weight h, uint64_t x_dptr, int x_dtype, uint64_t bias_dptr,
                     uint64_t out_dptr, uint32_t m) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->capturing || ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_linear_static during a recording");
  const Weight* w = find_weight(ctx, h);
  const int rc = check_linear_args(ctx, w, x_dptr, x_dtype, bias_dptr, out_dptr);
  if (rc != KQ_OK) return rc;
  DeviceGuard guard(ctx->device);
  const kq::LinearTarget target{w, reinterpret_cast<const float*>(bias_dptr), reinterpret_cast<float*>(out_dptr)};
  const char* why = "";
  int device_status = 0;
  cudaError_t e = kq::linear_static(env_of(ctx), target, reinterpret_cast<const void*>(x_dptr), x_dtype, m, &why,
                                    &device_status);
  if (e != cudaSuccess) {
    if (why[0] != 0) return fail(ctx, KQ_ERR_UNSUPPORTED, "kq_linear_static: %s", why);
    return cuda_fail(ctx, e, "kq_linear_static");
  }
  ctx->launches += 1;
  if (device_status != 0)
    return fail(ctx, KQ_ERR_TIMEOUT, "kq_linear_static: a bounded wait inside the kernel gave up; the output is not valid");
  return KQ_OK;
}

int kq_linear_tc(kq_ctx* ctx, uint32_t count, const kq_weight* handles, uint64_t x_dptr, int x_dtype,
                 const uint64_t* bias_dptr, const uint64_t* out_dptr, uint32_t m) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_linear_tc cannot be recorded into a fused plan");
  if (count < 1 || count > static_cast<uint32_t>(kq::kMaxMulti) || !handles || !bias_dptr || !out_dptr)
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_tc: 1..%d weights with their bias and output pointers", kq::kMaxMulti);
  kq::LinearTarget targets[kq::kMaxMulti];
  for (uint32_t i = 0; i < count; ++i) {
    const Weight* w = find_weight(ctx, handles[i]);
    const int rc = check_linear_args(ctx, w, x_dptr, x_dtype, bias_dptr[i], out_dptr[i]);
    if (rc != KQ_OK) return rc;
    targets[i] = kq::LinearTarget{w, reinterpret_cast<const float*>(bias_dptr[i]), reinterpret_cast<float*>(out_dptr[i])};
  }
  const kq::LaunchEnv env = env_of(ctx);
  if (!kq::qgemv_i4_tc_supports(static_cast<int>(count), targets, x_dtype, m, env.sm_count))
    return fail(ctx, KQ_ERR_UNSUPPORTED,
                "kq_linear_tc: tiled int4 / group-32 weights of one k and scale type, 5..16 binary16 rows or 5..8 f32 / bf16 "
                "rows, and a k whose activation image fits shared memory (got m=%u, k=%u)", m, targets[0].w ? targets[0].w->k : 0u);
  DeviceGuard guard(ctx->device);
  int launched = 0;
  cudaError_t e = kq::launch_qgemv_i4_tc(env, static_cast<int>(count), targets, reinterpret_cast<const void*>(x_dptr), x_dtype, m,
                                         &launched);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "kq_linear_tc");
  ctx->launches += launched;
  return KQ_OK;
}

int kq_embedding(kq_ctx* ctx, kq_weight h, uint64_t index_dptr, uint32_t rows, uint64_t out_dptr) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_embedding cannot be recorded into a fused plan");
  const Weight* w = find_weight(ctx, h);
  if (!w) return fail(ctx, KQ_ERR_BAD_ARG, "kq_embedding: unknown weight");
  if (rows != 0 && w->k != 0 && (!index_dptr || !out_dptr)) return fail(ctx, KQ_ERR_BAD_ARG, "kq_embedding: null device pointer");
  if (rows == 0 || w->k == 0) return KQ_OK;
  DeviceGuard guard(ctx->device);
  cudaError_t e = kq::launch_embedding(env_of(ctx), *w, reinterpret_cast<const int*>(index_dptr), rows,
                                       reinterpret_cast<float*>(out_dptr));
  if (e != cudaSuccess) return cuda_fail(ctx, e, "embedding launch");
  ctx->launches += 1;
  return KQ_OK;
}

int kq_quantize_rows(kq_ctx* ctx, uint64_t x_dptr, uint32_t rows, uint32_t dim, uint64_t q_dptr, uint64_t scale_dptr) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_quantize_rows cannot be recorded into a fused plan");
  if (rows != 0 && dim != 0 && (!x_dptr || !q_dptr || !scale_dptr))
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_quantize_rows: null device pointer");
  if (rows == 0 || dim == 0) return KQ_OK;
  DeviceGuard guard(ctx->device);
  cudaError_t e = kq::launch_quantize_rows(ctx->stream, reinterpret_cast<const float*>(x_dptr), rows, dim,
                                           reinterpret_cast<int8_t*>(q_dptr), reinterpret_cast<float*>(scale_dptr),
                                           nullptr, nullptr);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "quantize_rows launch");
  ctx->launches += 1;
  return KQ_OK;
}

int kq_linear_a8(kq_ctx* ctx, kq_weight h, uint64_t xq_dptr, uint64_t xs_dptr, uint64_t bias_dptr, uint64_t out_dptr,
                 uint32_t m) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_linear_a8 cannot be recorded into a fused plan");
  const Weight* w = find_weight(ctx, h);
  if (!w) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_a8: unknown weight");
  if (m != 0 && w->n != 0 && (!xq_dptr || !xs_dptr || !bias_dptr || !out_dptr))
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_a8: null device pointer (bias is required: the op's arity is 3)");
  // The int8 variant reduces the whole k range in int32: |sum| <= k * 127^2
  // (LINEAR_I8A8_MAX_K, packages/runtime/src/kernels/linear-i8a8.ts:121).  The int4 variant
  // flushes per group and has no such gate.
  if (w->storage == KQ_STORAGE_I8 && w->k > 131072u)
    return fail(ctx, KQ_ERR_UNSUPPORTED, "kq_linear_a8: k=%u exceeds the int32 reduction gate 131072", w->k);
  if (m == 0 || w->n == 0) return KQ_OK;
  DeviceGuard guard(ctx->device);
  const bool tiled = w->layout == kq::kLayoutTiledI4 || w->layout == kq::kLayoutTiledI8;
  int* row_sum = nullptr;
  int* group_sum = nullptr;
  int launched = 0;
  if (tiled) {
    const uint64_t need = (static_cast<uint64_t>(m) * (w->k / 32) + m) * sizeof(int);
    if (need > ctx->idot_sums_bytes) {
      if (ctx->capturing) return fail(ctx, KQ_ERR_STATE, "kq_linear_a8: scratch must grow; call once outside the recording first");
      if (ctx->idot_sums) cudaFree(ctx->idot_sums);
      ctx->idot_sums = nullptr;
      ctx->idot_sums_bytes = 0;
      KQ_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&ctx->idot_sums), need));
      ctx->idot_sums_bytes = need;
    }
    row_sum = ctx->idot_sums;
    group_sum = ctx->idot_sums + m;
    cudaError_t e = kq::launch_xq_sums(ctx->stream, reinterpret_cast<const int8_t*>(xq_dptr), m, w->k, row_sum, group_sum);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "xq_sums launch");
    launched += 1;
  }
  cudaError_t e = kq::launch_linear_idot(ctx->stream, *w, reinterpret_cast<const int8_t*>(xq_dptr),
                                         reinterpret_cast<const float*>(xs_dptr), row_sum, group_sum,
                                         reinterpret_cast<const float*>(bias_dptr), reinterpret_cast<float*>(out_dptr),
                                         m, &launched);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "linear_a8 launch");
  ctx->launches += launched;
  return KQ_OK;
}

int kq_comm_create(kq_ctx* ctx, uint32_t rank, uint32_t world, uint64_t max_bytes, uint8_t* out_handle) {
  if (!ctx || !out_handle) return fail(ctx, KQ_ERR_BAD_ARG, "kq_comm_create: null argument");
  if (ctx->comm) return fail(ctx, KQ_ERR_STATE, "kq_comm_create: this context already has an exchange");
  DeviceGuard guard(ctx->device);
  cudaError_t e = cudaSuccess;
  const char* why = "";
  ctx->comm = kq::comm_create(rank, world, max_bytes, out_handle, &e, &why);
  if (!ctx->comm) {
    if (why[0] != 0) return fail(ctx, KQ_ERR_BAD_ARG, "kq_comm_create: %s", why);
    return cuda_fail(ctx, e, "kq_comm_create");
  }
  return KQ_OK;
}

int kq_comm_connect(kq_ctx* ctx, const uint8_t* all_handles) {
  if (!ctx || !all_handles) return fail(ctx, KQ_ERR_BAD_ARG, "kq_comm_connect: null argument");
  if (!ctx->comm) return fail(ctx, KQ_ERR_STATE, "kq_comm_connect before kq_comm_create");
  DeviceGuard guard(ctx->device);
  cudaError_t e = kq::comm_connect(ctx->comm, all_handles);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "kq_comm_connect (cudaIpcOpenMemHandle)");
  return KQ_OK;
}

int kq_all_reduce(kq_ctx* ctx, uint64_t dptr, uint64_t count) {
  if (!ctx || !dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_all_reduce: null argument");
  if (!kq::comm_connected(ctx->comm)) return fail(ctx, KQ_ERR_STATE, "kq_all_reduce before kq_comm_connect");
  if (dptr & 15u) return fail(ctx, KQ_ERR_BAD_ARG, "kq_all_reduce: the vector must be 16-byte aligned");
  if (count * sizeof(float) > kq::comm_max_bytes(ctx->comm))
    return fail(ctx, KQ_ERR_SHAPE, "kq_all_reduce: %llu bytes exceed the %llu the exchange was created for",
                (unsigned long long)(count * sizeof(float)), (unsigned long long)kq::comm_max_bytes(ctx->comm));
  if (count == 0) return KQ_OK;
  DeviceGuard guard(ctx->device);
  cudaError_t e = kq::comm_all_reduce(ctx->comm, ctx->stream, reinterpret_cast<float*>(dptr), count);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "kq_all_reduce launch");
  ctx->launches += 1;
  return KQ_OK;
}

int kq_linear_reduce(kq_ctx* ctx, kq_weight h, uint64_t x_dptr, int x_dtype, uint64_t bias_dptr, uint64_t out_dptr,
                     uint32_t m) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_linear_reduce cannot be recorded into a fused plan");
  if (!kq::comm_connected(ctx->comm)) return fail(ctx, KQ_ERR_STATE, "kq_linear_reduce before kq_comm_connect");
  const Weight* w = find_weight(ctx, h);
  const int rc = check_linear_args(ctx, w, x_dptr, x_dtype, bias_dptr, out_dptr);
  if (rc != KQ_OK) return rc;
  if (out_dptr & 15u) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_reduce: out must be 16-byte aligned");
  const uint64_t count = static_cast<uint64_t>(m) * w->n;
  if (count * sizeof(float) > kq::comm_max_bytes(ctx->comm))
    return fail(ctx, KQ_ERR_SHAPE, "kq_linear_reduce: %llu bytes exceed the %llu the exchange was created for",
                (unsigned long long)(count * sizeof(float)), (unsigned long long)kq::comm_max_bytes(ctx->comm));
  if (count == 0) return KQ_OK;
  DeviceGuard guard(ctx->device);
  // One kernel: the group-packed GEMV adds the ranks' partial sums in its epilogue.
  if (w->layout == kq::kLayoutTiledI4 && kq::qgemv_i4_supports(*w, m)) {
    kq::LaunchEnv env = env_of(ctx);
    env.fused = kq::comm_fused_view(ctx->comm);
    const kq::LinearTarget target{w, reinterpret_cast<const float*>(bias_dptr), reinterpret_cast<float*>(out_dptr)};
    int launched = 0;
    cudaError_t e = kq::launch_qgemv_i4(env, 1, &target, reinterpret_cast<const void*>(x_dptr), x_dtype, m, &launched);
    if (e == cudaSuccess) {
      ctx->launches += launched;
      return KQ_OK;
    }
    if (e != cudaErrorNotSupported) return cuda_fail(ctx, e, "fused linear + exchange launch");
    (void)cudaGetLastError();
  }
  // Two steps: the linear with the bias on rank 0 only, then the all-reduce.
  uint64_t bias_here = bias_dptr;
  if (kq::comm_rank(ctx->comm) != 0) {
    if (w->n > ctx->zero_bias_count) {
      if (ctx->capturing) return fail(ctx, KQ_ERR_STATE, "kq_linear_reduce: scratch must grow; call once outside the recording first");
      if (ctx->zero_bias) cudaFree(ctx->zero_bias);
      ctx->zero_bias = nullptr;
      ctx->zero_bias_count = 0;
      KQ_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&ctx->zero_bias), static_cast<size_t>(w->n) * sizeof(float)));
      KQ_CUDA(ctx, cudaMemset(ctx->zero_bias, 0, static_cast<size_t>(w->n) * sizeof(float)));
      ctx->zero_bias_count = w->n;
    }
    bias_here = reinterpret_cast<uint64_t>(ctx->zero_bias);
  }
  const int rc2 = run_linear(ctx, 1, &h, x_dptr, x_dtype, &bias_here, &out_dptr, m);
  if (rc2 != KQ_OK) return rc2;
  cudaError_t e = kq::comm_all_reduce(ctx->comm, ctx->stream, reinterpret_cast<float*>(out_dptr), count);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "kq_linear_reduce: all-reduce launch");
  ctx->launches += 1;
  return KQ_OK;
}

// Grows one of the context's lazily allocated scratch buffers (never during a graph capture).
static int grow_scratch(kq_ctx* ctx, float** buf, uint64_t* have, uint64_t need, const char* who) {
  if (need <= *have) return KQ_OK;
  if (ctx->capturing) return fail(ctx, KQ_ERR_STATE, "%s: scratch must grow; call once outside the recording first", who);
  if (*buf) cudaFree(*buf);
  *buf = nullptr;
  *have = 0;
  KQ_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(buf), need));
  *have = need;
  return KQ_OK;
}

int kq_rms_norm(kq_ctx* ctx, uint64_t x_dptr, uint64_t weight_dptr, float eps, uint64_t out_dptr, uint32_t rows,
                uint32_t dim) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_rms_norm cannot be recorded into a fused plan (use kq_linear_fused)");
  // packages/runtime/src/kernels/rms-norm.ts:100-117: dim >= 1, eps finite and positive
  if (dim < 1) return fail(ctx, KQ_ERR_SHAPE, "kq_rms_norm: dim must be positive");
  if (!(eps > 0.0f) || !(eps < __builtin_inff())) return fail(ctx, KQ_ERR_BAD_ARG, "kq_rms_norm: eps must be finite and positive");
  if (rows == 0) return KQ_OK;
  if (!x_dptr || !weight_dptr || !out_dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_rms_norm: null device pointer");
  DeviceGuard guard(ctx->device);
  cudaError_t e = kq::launch_rms_norm(env_of(ctx), reinterpret_cast<const float*>(x_dptr), reinterpret_cast<const float*>(weight_dptr),
                                      eps, reinterpret_cast<float*>(out_dptr), rows, dim);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "rms_norm launch");
  ctx->launches += 1;
  return KQ_OK;
}

int kq_silu_mul(kq_ctx* ctx, uint64_t gate_dptr, uint64_t up_dptr, uint64_t out_dptr, uint64_t count) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_silu_mul cannot be recorded into a fused plan (use kq_linear_fused)");
  if (count == 0) return KQ_OK;
  if (!gate_dptr || !up_dptr || !out_dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_silu_mul: null device pointer");
  DeviceGuard guard(ctx->device);
  cudaError_t e = kq::launch_silu_mul(env_of(ctx), reinterpret_cast<const float*>(gate_dptr), reinterpret_cast<const float*>(up_dptr),
                                      reinterpret_cast<float*>(out_dptr), count);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "silu_mul launch");
  ctx->launches += 1;
  return KQ_OK;
}

int kq_add(kq_ctx* ctx, uint64_t a_dptr, uint64_t b_dptr, uint64_t out_dptr, uint64_t count) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_add cannot be recorded into a fused plan (use kq_linear_fused)");
  if (count == 0) return KQ_OK;
  if (!a_dptr || !b_dptr || !out_dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_add: null device pointer");
  DeviceGuard guard(ctx->device);
  cudaError_t e = kq::launch_add(env_of(ctx), reinterpret_cast<const float*>(a_dptr), reinterpret_cast<const float*>(b_dptr),
                                 reinterpret_cast<float*>(out_dptr), count);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "add launch");
  ctx->launches += 1;
  return KQ_OK;
}

int kq_linear_fused(kq_ctx* ctx, uint32_t count, const kq_weight* w, uint64_t x_dptr, int x_dtype,
                    uint64_t norm_weight_dptr, float norm_eps, const uint64_t* bias_dptr, uint64_t residual_dptr,
                    const uint64_t* out_dptr, uint32_t m, uint32_t flags) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (!w || !bias_dptr || !out_dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: null argument");
  if (flags & ~static_cast<uint32_t>(KQ_FUSE_SWIGLU | KQ_FUSE_REDUCE))
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: unknown flag bits 0x%x", flags);
  const bool swiglu = (flags & KQ_FUSE_SWIGLU) != 0, reduce = (flags & KQ_FUSE_REDUCE) != 0;
  if (count < 1 || count > (uint32_t)kq::kMaxMulti)
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: count %u outside 1..%d", count, kq::kMaxMulti);
  if (swiglu && (count != 2 || reduce || residual_dptr))
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: the SiLU gate takes two weights (gate, up) and combines with a norm only");
  if ((reduce || residual_dptr) && count != 1)
    return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: a residual or a cross-rank reduce goes with a single weight");
  if (norm_weight_dptr) {
    if (x_dtype != KQ_F32) return fail(ctx, KQ_ERR_UNSUPPORTED, "kq_linear_fused: the norm takes f32 activations (rms_norm is an f32 op)");
    if (!(norm_eps > 0.0f) || !(norm_eps < __builtin_inff()))
      return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: eps must be finite and positive");
    if (norm_weight_dptr & 15u) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: the norm weight must be 16-byte aligned");
  }
  const Weight* w0 = find_weight(ctx, w[0]);
  if (!w0) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: unknown weight handle");
  if (swiglu) {
    const Weight* w1 = find_weight(ctx, w[1]);
    if (!w1 || w1->n != w0->n || w1->k != w0->k)
      return fail(ctx, KQ_ERR_SHAPE, "kq_linear_fused: gate and up weights differ in shape");
  }
  if (reduce && !kq::comm_connected(ctx->comm)) return fail(ctx, KQ_ERR_STATE, "kq_linear_fused: KQ_FUSE_REDUCE before kq_comm_connect");
  if (residual_dptr && (residual_dptr & 3u)) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: residual must be 4-byte aligned");

  if (ctx->recording) {
    kq::LinearFusion fusion;
    fusion.norm_weight = reinterpret_cast<const float*>(norm_weight_dptr);
    fusion.norm_eps = norm_eps;
    fusion.residual = reinterpret_cast<const float*>(residual_dptr);
    fusion.swiglu = swiglu;
    fusion.reduce = reduce;
    // the gate pair has one output; the recorder checks one pointer per weight
    const uint64_t gate_outs[2] = {out_dptr[0], out_dptr[0]};
    return run_linear(ctx, count, w, x_dptr, x_dtype, bias_dptr, swiglu ? gate_outs : out_dptr, m, &fusion);
  }
  if (m == 0) return KQ_OK;
  DeviceGuard guard(ctx->device);
  // Outside a plan: the same arithmetic as a sequence of kernels — except where the GEMV takes
  // the norm and the residual into its own launches (five and more rows, tiled int4 weights).
  {
    kq::LinearTarget probe[kq::kMaxMulti];
    bool known = true;
    for (uint32_t i = 0; i < count; ++i) {
      probe[i] = kq::LinearTarget{find_weight(ctx, w[i]), nullptr, nullptr};
      known = known && probe[i].w != nullptr;
    }
    if (known && !reduce &&
        kq::qgemv_i4_fuses_neighbours(static_cast<int>(count), probe, x_dtype, m) && (norm_weight_dptr || residual_dptr)) {
      int rc;
      if (swiglu) {
        const uint64_t each = static_cast<uint64_t>(m) * w0->n;
        rc = grow_scratch(ctx, &ctx->fused_gu, &ctx->fused_gu_bytes, 2 * each * sizeof(float), "kq_linear_fused");
        if (rc != KQ_OK) return rc;
        if (!out_dptr[0]) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: out is null");
        const uint64_t outs[2] = {reinterpret_cast<uint64_t>(ctx->fused_gu), reinterpret_cast<uint64_t>(ctx->fused_gu + each)};
        ctx->nb_norm_weight = reinterpret_cast<const float*>(norm_weight_dptr);
        ctx->nb_norm_eps = norm_eps;
        rc = run_linear(ctx, 2, w, x_dptr, x_dtype, bias_dptr, outs, m);
        ctx->nb_norm_weight = nullptr;
        if (rc != KQ_OK) return rc;
        cudaError_t e = kq::launch_silu_mul(env_of(ctx), ctx->fused_gu, ctx->fused_gu + each, reinterpret_cast<float*>(out_dptr[0]), each);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "silu_mul launch");
        ctx->launches += 1;
        return KQ_OK;
      }
      ctx->nb_norm_weight = reinterpret_cast<const float*>(norm_weight_dptr);
      ctx->nb_norm_eps = norm_eps;
      ctx->nb_residual = reinterpret_cast<const float*>(residual_dptr);
      rc = run_linear(ctx, count, w, x_dptr, x_dtype, bias_dptr, out_dptr, m);
      ctx->nb_norm_weight = nullptr;
      ctx->nb_residual = nullptr;
      return rc;
    }
  }
  uint64_t x_eff = x_dptr;
  if (norm_weight_dptr) {
    if (!x_dptr) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: x is null");
    const int rc = grow_scratch(ctx, &ctx->fused_xn, &ctx->fused_xn_bytes, static_cast<uint64_t>(m) * w0->k * sizeof(float), "kq_linear_fused");
    if (rc != KQ_OK) return rc;
    cudaError_t e = kq::launch_rms_norm(env_of(ctx), reinterpret_cast<const float*>(x_dptr), reinterpret_cast<const float*>(norm_weight_dptr),
                                        norm_eps, ctx->fused_xn, m, w0->k);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "rms_norm launch");
    ctx->launches += 1;
    x_eff = reinterpret_cast<uint64_t>(ctx->fused_xn);
  }
  if (swiglu) {
    const uint64_t each = static_cast<uint64_t>(m) * w0->n;
    const int rc = grow_scratch(ctx, &ctx->fused_gu, &ctx->fused_gu_bytes, 2 * each * sizeof(float), "kq_linear_fused");
    if (rc != KQ_OK) return rc;
    if (!out_dptr[0]) return fail(ctx, KQ_ERR_BAD_ARG, "kq_linear_fused: out is null");
    const uint64_t outs[2] = {reinterpret_cast<uint64_t>(ctx->fused_gu), reinterpret_cast<uint64_t>(ctx->fused_gu + each)};
    const int rc2 = run_linear(ctx, 2, w, x_eff, x_dtype, bias_dptr, outs, m);
    if (rc2 != KQ_OK) return rc2;
    cudaError_t e = kq::launch_silu_mul(env_of(ctx), ctx->fused_gu, ctx->fused_gu + each, reinterpret_cast<float*>(out_dptr[0]), each);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "silu_mul launch");
    ctx->launches += 1;
    return KQ_OK;
  }
  // With a residual the linear lands in scratch first: the residual may be the output buffer.
  uint64_t lin_out = out_dptr[0];
  if (residual_dptr) {
    const int rc = grow_scratch(ctx, &ctx->fused_gu, &ctx->fused_gu_bytes, static_cast<uint64_t>(m) * w0->n * sizeof(float), "kq_linear_fused");
    if (rc != KQ_OK) return rc;
    lin_out = reinterpret_cast<uint64_t>(ctx->fused_gu);
  }
  const int rc = reduce ? kq_linear_reduce(ctx, w[0], x_eff, x_dtype, bias_dptr[0], lin_out, m)
                        : run_linear(ctx, count, w, x_eff, x_dtype, bias_dptr, residual_dptr ? &lin_out : out_dptr, m);
  if (rc != KQ_OK) return rc;
  if (residual_dptr) {
    cudaError_t e = kq::launch_add(env_of(ctx), ctx->fused_gu, reinterpret_cast<const float*>(residual_dptr),
                                   reinterpret_cast<float*>(out_dptr[0]), static_cast<uint64_t>(m) * w0->n);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "residual add launch");
    ctx->launches += 1;
  }
  return KQ_OK;
}

int kq_plan_begin(kq_ctx* ctx) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  if (ctx->capturing || ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_plan_begin: a recording is already open");
  ctx->recording = kq::plan_create();
  ctx->recording_refusal.clear();
  return KQ_OK;
}

int kq_plan_end(kq_ctx* ctx, kq_plan* out) {
  if (!ctx || !out) return fail(ctx, KQ_ERR_BAD_ARG, "kq_plan_end: null argument");
  if (!ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_plan_end without kq_plan_begin");
  *out = 0;
  kq::Plan* plan = ctx->recording;
  ctx->recording = nullptr;
  DeviceGuard guard(ctx->device);
  if (!ctx->recording_refusal.empty()) {
    kq::plan_destroy(plan);
    return fail(ctx, KQ_ERR_UNSUPPORTED, "the plan cannot be fused: %s (record it with kq_graph_begin instead)",
                ctx->recording_refusal.c_str());
  }
  const char* why = "";
  kq::LaunchEnv env = env_of(ctx);
  env.fused = kq::comm_fused_view(ctx->comm);
  cudaError_t e = kq::plan_finalize(plan, env, &why);
  if (e != cudaSuccess) {
    kq::plan_destroy(plan);
    if (why[0] != 0) return fail(ctx, KQ_ERR_UNSUPPORTED, "%s", why);
    return cuda_fail(ctx, e, "kq_plan_end");
  }
  const uint64_t handle = ctx->next_handle++;
  ctx->plans[handle] = plan;
  *out = handle;
  return KQ_OK;
}

int kq_plan_launch(kq_ctx* ctx, kq_plan plan) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  auto it = ctx->plans.find(plan);
  if (it == ctx->plans.end()) return fail(ctx, KQ_ERR_BAD_ARG, "kq_plan_launch: unknown plan handle");
  if (ctx->capturing || ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_plan_launch during a recording");
  DeviceGuard guard(ctx->device);
  int launched = 0;
  cudaError_t e = kq::plan_launch(it->second, env_of(ctx), &launched);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "kq_plan_launch");
  ctx->launches += launched;
  return KQ_OK;
}

int kq_plan_profile(kq_ctx* ctx, kq_plan plan, uint64_t* stamps, uint64_t capacity, uint32_t* out_ctas, uint32_t* out_ops,
                    uint32_t* out_slots) {
  if (!ctx || !out_ctas || !out_ops || !out_slots) return fail(ctx, KQ_ERR_BAD_ARG, "kq_plan_profile: null argument");
  auto it = ctx->plans.find(plan);
  if (it == ctx->plans.end()) return fail(ctx, KQ_ERR_BAD_ARG, "kq_plan_profile: unknown plan handle");
  if (ctx->capturing || ctx->recording) return fail(ctx, KQ_ERR_STATE, "kq_plan_profile during a recording");
  if (!kq::plan_is_paired(it->second))
    return fail(ctx, KQ_ERR_UNSUPPORTED, "kq_plan_profile: only the paired kernel (one or two rows) leaves phase stamps");
  const uint32_t ctas = kq::plan_grid(it->second), ops = kq::plan_op_count(it->second), slots = kq::plan_trace_slots();
  *out_ctas = ctas;
  *out_ops = ops;
  *out_slots = slots;
  const uint64_t need = static_cast<uint64_t>(ctas) * ops * slots;
  if (!stamps) return KQ_OK;  // size query
  if (capacity < need) return fail(ctx, KQ_ERR_SHAPE, "kq_plan_profile: %llu stamps needed, room for %llu", (unsigned long long)need,
                                   (unsigned long long)capacity);
  DeviceGuard guard(ctx->device);
  unsigned long long* dev = nullptr;
  KQ_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&dev), need * sizeof(unsigned long long)));
  cudaError_t e = cudaMemsetAsync(dev, 0, need * sizeof(unsigned long long), ctx->stream);
  int launched = 0;
  if (e == cudaSuccess) e = kq::plan_launch(it->second, env_of(ctx), &launched, dev);
  if (e == cudaSuccess) e = cudaMemcpyAsync(stamps, dev, need * sizeof(unsigned long long), cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaFree(dev);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "kq_plan_profile");
  ctx->launches += launched;
  return KQ_OK;
}

int kq_plan_free(kq_ctx* ctx, kq_plan plan) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  auto it = ctx->plans.find(plan);
  if (it == ctx->plans.end()) return fail(ctx, KQ_ERR_BAD_ARG, "kq_plan_free: unknown plan handle");
  DeviceGuard guard(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  kq::plan_destroy(it->second);
  ctx->plans.erase(it);
  return KQ_OK;
}

int kq_timer_start(kq_ctx* ctx) {
  if (!ctx) return KQ_ERR_BAD_ARG;
  DeviceGuard guard(ctx->device);
  KQ_CUDA(ctx, cudaEventRecord(ctx->ev_start, ctx->stream));
  return KQ_OK;
}

int kq_timer_stop(kq_ctx* ctx, float* out_ms) {
  if (!ctx || !out_ms) return fail(ctx, KQ_ERR_BAD_ARG, "kq_timer_stop: null argument");
  DeviceGuard guard(ctx->device);
  KQ_CUDA(ctx, cudaEventRecord(ctx->ev_stop, ctx->stream));
  KQ_CUDA(ctx, cudaEventSynchronize(ctx->ev_stop));
  KQ_CUDA(ctx, cudaEventElapsedTime(out_ms, ctx->ev_start, ctx->ev_stop));
  return KQ_OK;
}

uint64_t kq_launch_count(kq_ctx* ctx) { return ctx ? ctx->launches : 0; }

}  // extern "C"
