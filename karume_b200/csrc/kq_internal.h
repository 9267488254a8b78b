// Host-side declarations shared by the translation units of libkq.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kq.h"

namespace kq {

enum Layout : int {
  kLayoutNative = 0,  // payload and scale exactly as uploaded (row-major)
  kLayoutTiledI4 = 1,  // chunked int4 layout described in kq_common.cuh (group size 32)
  kLayoutTiledI8 = 2   // chunked int8 layout described in kq_common.cuh (scales stay [n])
};

struct Weight {
  int storage = 0;      // kq_storage
  int scale_dtype = 0;  // kq_dtype (KQ_F32 or KQ_F16)
  uint32_t n = 0, k = 0, group_size = 0;
  int layout = kLayoutNative;
  void* data = nullptr;   // native: payload; tiled: interleaved chunks (payload + scales)
  void* scale = nullptr;  // native: scales; tiled: nullptr
  uint64_t payload_bytes = 0, scale_bytes = 0;
};

// One launch's worth of "several weights, same x" (kq_linear_multi).
constexpr int kMaxMulti = 4;

struct LinearTarget {
  const Weight* w;
  const float* bias;
  float* out;
};

// The neighbours of a linear that kq_linear_fused attaches to it.
struct LinearFusion {
  const float* norm_weight = nullptr;  // [k] f32: x is rms-normalised first
  float norm_eps = 0.0f;
  const float* residual = nullptr;     // [m, n] f32 added to the single output
  bool swiglu = false;                 // two weights (gate, up) -> one output silu(gate) * up
  bool reduce = false;                 // row-parallel shard: add the outputs across ranks
};

// Device-side view of the tensor-parallel exchange area a row-parallel GEMV uses to add its
// partial sums across ranks inside its own epilogue (kq_comm.cu owns the memory).
constexpr int kFusedMaxWorld = 8;
constexpr uint32_t kFusedMaxCtas = 1024;          // largest grid the fused exchange accepts
constexpr uint64_t kFusedSlotBytes = 64 * 1024;   // m * n entries of 8 bytes {value, epoch} per source rank and parity
struct FusedCommDev {
  uint8_t* base[kFusedMaxWorld];  // every rank's allocation (own included), peer-mapped
  uint32_t rank, world;
  uint64_t flags_off;   // reserved
  uint64_t data_off;    // [2][world][kFusedSlotBytes]: {value, epoch} entries pushed by peers
  unsigned int* epoch;  // local: advanced by the last CTA of every fused launch
  unsigned int* done;   // local: CTAs that finished their epilogue
  int* status;          // host-mapped: non-zero once a bounded wait gave up
};

// What a launcher remembers about a kernel — attributes set before its first launch, limits learnt
// from the device — belongs to a device, not to the process: a host may drive several GPUs from
// one process.  slot() is the entry of the calling thread's current device (nullptr if that
// cannot be told).
template <typename T, int kDevices = 64>
struct PerDevice {
  T value[kDevices] = {};
  T* slot() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kDevices) return nullptr;
    return &value[device];
  }
};

struct LaunchEnv {
  cudaStream_t stream;
  bool overlap;          // programmatic dependent launch
  void* workspace;       // split-K partial sums
  uint64_t workspace_bytes;
  unsigned int* counters;  // split-K arrival counters (zero between launches)
  uint32_t counter_count;
  int sm_count;
  const FusedCommDev* fused = nullptr;  // non-null: add the output across ranks in the epilogue
  int* status = nullptr;  // device-visible word a kernel sets when one of its bounded waits gives up
  // Neighbours the wide GEMV (5..16 activation rows, one weight or several) takes into its own
  // launches when qgemv_i4_fuses_neighbours() says so: an rms_norm of the f32 activations in its
  // staging pre-kernel and a residual [m, n] (single weight; may alias the output) in its stores.
  const float* norm_weight = nullptr;
  float norm_eps = 0.0f;
  const float* residual = nullptr;
};

// Generic kernels: any shape the storage contract allows, native layout.
cudaError_t launch_linear_generic(const LaunchEnv& env, const Weight& w, const void* x, int x_dtype,
                                  const float* bias, float* out, uint32_t m);
cudaError_t launch_dequant(const LaunchEnv& env, const Weight& w, float* out);
cudaError_t launch_embedding(const LaunchEnv& env, const Weight& w, const int* index, uint32_t rows, float* out);

// Tiled int4 layout.
bool tiled_i4_eligible(int storage, uint32_t n, uint32_t k, uint32_t group_size);
cudaError_t launch_repack_i4(cudaStream_t stream, const uint8_t* payload, const void* scale,
                             int scale_dtype, uint32_t n, uint32_t k, uint8_t* tiled);

// Tiled int8 layout.
bool tiled_i8_eligible(int storage, uint32_t n, uint32_t k);
cudaError_t launch_repack_i8(cudaStream_t stream, const uint8_t* payload, uint32_t n, uint32_t k, uint8_t* tiled);
cudaError_t launch_qgemv_i8(const LaunchEnv& env, const LinearTarget& target, const void* x, int x_dtype,
                            uint32_t m);

// Tensor-core GEMV for the tiled int4 layout, m <= 16.  Returns cudaErrorInvalidValue
// when the request needs more workspace than the context owns.
bool qgemv_i4_supports(const Weight& w, uint32_t m);
bool qgemv_i4_fuses_neighbours(int count, const LinearTarget* targets, int x_dtype, uint32_t m);
cudaError_t launch_qgemv_i4(const LaunchEnv& env, int count, const LinearTarget* targets,
                            const void* x, int x_dtype, uint32_t m, int* launches);

// The same on the tcgen05 tensor cores (kq_qgemv_i4_tc.cu): 5..16 binary16 rows or 5..8 f32 /
// bf16 rows.  Needs env.status.
bool qgemv_i4_tc_supports(int count, const LinearTarget* targets, int x_dtype, uint32_t m, int sm_count);
cudaError_t launch_qgemv_i4_tc(const LaunchEnv& env, int count, const LinearTarget* targets, const void* x, int x_dtype,
                               uint32_t m, int* launches);

}  // namespace kq

// ---- tcgen05 prefill GEMM (kq_qgemm_i4.cu): tiled int4 weights, bf16 activations, m > 16
namespace kq {
bool qgemm_i4_supports(const Weight& w, int x_dtype, uint32_t m);
// The same GEMM over a tiled int8 weight (launch_qgemm_i4 takes both storages).
bool qgemm_i8_supports(const Weight& w, int x_dtype, uint32_t m);
cudaError_t launch_qgemm_i4(const LaunchEnv& env, const LinearTarget& target, const void* x, uint32_t m,
                            int* status_word, int* extra_launches);
// The same for f32 and binary16 activations (kq_qgemm_i4_x32.cu): both operands as two bf16 numbers.
bool qgemm_i4_x32_supports(const Weight& w, int x_dtype, uint32_t m, uint64_t workspace_bytes);
cudaError_t launch_qgemm_i4_x32(const LaunchEnv& env, const LinearTarget& target, const void* x, int x_dtype, uint32_t m,
                                int* status_word, int* launches);
}  // namespace kq

// ---- error reporting shared with kq_container.cu (kq_api.cu) ------------------------------
#include <string>
namespace kq {
void set_global_error(const std::string& message);              // read back by kq_last_error(NULL)
int ctx_fail(kq_ctx* ctx, int code, const std::string& message);  // stores the message, returns the code
}  // namespace kq

// ---- fused plans (kq_plan.cu) -------------------------------------------------------
namespace kq {
struct Plan;
Plan* plan_create();
void plan_destroy(Plan* plan);
const char* plan_add_copy(Plan* plan, bool to_device, void* device, void* host, uint64_t bytes);
const char* plan_add_linear(Plan* plan, int count, const LinearTarget* targets, const void* x, int x_dtype,
                            uint32_t m, const LinearFusion& fusion);
uint32_t plan_op_count(const Plan* plan);
cudaError_t plan_finalize(Plan* plan, const LaunchEnv& env, const char** why);
cudaError_t plan_launch(Plan* plan, const LaunchEnv& env, int* launches, unsigned long long* trace = nullptr);
uint32_t plan_grid(const Plan* plan);
bool plan_is_paired(const Plan* plan);
uint32_t plan_trace_slots();
int plan_take_status(Plan* plan);
// One linear through the fused kernel with every scratch byte in a static device array.
cudaError_t linear_static(const LaunchEnv& env, const LinearTarget& target, const void* x, int x_dtype,
                          uint32_t m, const char** why, int* device_status);
}  // namespace kq

// ---- peer-memory all-reduce (kq_comm.cu) ----------------------------------------------
namespace kq {
struct Comm;
Comm* comm_create(uint32_t rank, uint32_t world, uint64_t max_bytes, uint8_t* handle_out, cudaError_t* err,
                  const char** why);
cudaError_t comm_connect(Comm* c, const uint8_t* all_handles);
void comm_destroy(Comm* c);
bool comm_connected(const Comm* c);
uint64_t comm_max_bytes(const Comm* c);
cudaError_t comm_all_reduce(Comm* c, cudaStream_t stream, float* data, uint64_t count);
int comm_take_status(Comm* c);
const FusedCommDev* comm_fused_view(const Comm* c);
uint32_t comm_rank(const Comm* c);
}  // namespace kq

// ---- rms_norm, SiLU gate, residual add as kernels of their own (kq_fused_ops.cu) -----------
namespace kq {
cudaError_t launch_rms_norm(const LaunchEnv& env, const float* x, const float* weight, float eps, float* out,
                            uint32_t rows, uint32_t dim);
cudaError_t launch_silu_mul(const LaunchEnv& env, const float* gate, const float* up, float* out, uint64_t count);
cudaError_t launch_add(const LaunchEnv& env, const float* a, const float* b, float* out, uint64_t count);
}  // namespace kq

// ---- integer-dot linear (kq_idot.cu) ---------------------------------------------------
namespace kq {
cudaError_t launch_quantize_rows(cudaStream_t stream, const float* x, uint32_t rows, uint32_t dim, int8_t* q,
                                 float* scale, int* row_sum, int* group_sum);
cudaError_t launch_xq_sums(cudaStream_t stream, const int8_t* q, uint32_t rows, uint32_t dim, int* row_sum,
                           int* group_sum);
cudaError_t launch_linear_idot(cudaStream_t stream, const Weight& w, const int8_t* xq, const float* xs,
                               const int* row_sum, const int* group_sum, const float* bias, float* out,
                               uint32_t m, int* launches);
}  // namespace kq
