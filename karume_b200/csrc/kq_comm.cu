// Tensor-parallel exchange over NVLink peer memory: a one-shot, deterministic all-reduce
// for the small f32 vectors a row-parallel linear produces (16 KB .. 256 KB).
// karume is single-device; this has no reference counterpart.
//
// Every rank (one process per GPU) owns one device allocation laid out as
//     [flags: kMaxBlocks x kMaxWorld words][arrival epochs: kMaxBlocks words][slot 0][slot 1]
// exported with cudaIpcGetMemHandle and opened by every peer.  One all-reduce, per CTA b
// (each CTA owns a slice of the vector, no cross-CTA dependency):
//   1. copy the local slice into the local slot (epoch parity picks the slot);
//   2. system-scope fence, then store the epoch into flag[b][my rank] of EVERY peer;
//   3. wait (bounded) until flag[b][r] in local memory has reached the epoch for every r;
//   4. read the slice from every rank's slot with plain peer loads, add in rank order
//      0..world-1 (so all ranks produce the same bits) and write the result in place.
// Slot reuse is safe without a second barrier: a rank writes slot e%2 again at epoch e+2,
// i.e. after it has seen every peer arrive at epoch e+1, which a peer only does after it
// finished reading epoch e.  The epoch lives in device memory and is advanced by the
// kernel, so the launch can be captured in a CUDA graph and replayed.
// Waits are bounded; a wait that gives up sets a status word the host reports as
// KQ_ERR_TIMEOUT.  No multimem, no TMA: plain ld/st on peer pointers.
#include <cstring>

#include "kq_internal.h"

namespace kq {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxBlocks = 32;
constexpr int kCommThreads = 512;
constexpr uint32_t kCommSpinLimit = 1u << 22;
constexpr uint64_t kStripeVec = 1024;  // float4 per CTA stripe = 16 KB

struct CommParams {
  uint8_t* base[kMaxWorld];  // every rank's exported allocation (own included)
  uint32_t rank, world;
  uint64_t slot_bytes;
  float* data;      // in / out, f32
  uint64_t count;   // elements
  int* status;
};

__host__ __device__ inline uint64_t comm_flags_bytes() { return uint64_t(kMaxBlocks) * kMaxWorld * sizeof(unsigned int); }
__host__ __device__ inline uint64_t comm_epoch_off() { return comm_flags_bytes(); }
__host__ __device__ inline uint64_t comm_slot_off(uint64_t slot_bytes, uint32_t slot) {
  return comm_flags_bytes() + 256 + slot * slot_bytes;
}
// Area of the fused GEMV + exchange: [epoch, done | 256 B][flags][data], after the two slots.
inline uint64_t fused_off(uint64_t slot_bytes) { return (comm_slot_off(slot_bytes, 2) + 255) & ~uint64_t(255); }
inline uint64_t fused_flags_bytes() { return uint64_t(2) * kFusedMaxWorld * kFusedMaxCtas * sizeof(unsigned int); }
inline uint64_t fused_data_bytes() { return uint64_t(2) * kFusedMaxWorld * kFusedSlotBytes; }

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float4* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ float ld_peer_f32(const float* p) {
  float v;
  asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

__global__ void __launch_bounds__(kCommThreads)
all_reduce_kernel(const CommParams p) {
  const uint32_t b = blockIdx.x;
  uint8_t* mine = p.base[p.rank];
  unsigned int* epochs = reinterpret_cast<unsigned int*>(mine + comm_epoch_off());
  __shared__ unsigned int epoch_s;
  if (threadIdx.x == 0) epoch_s = epochs[b] + 1;
  __syncthreads();
  const unsigned int epoch = epoch_s;
  const uint32_t slot = epoch & 1u;

  // this CTA's slice, in float4 units: always the same 16 KB stripe of the slots, whatever
  // the size of the exchange, so the per-CTA epochs order every reuse of a stripe.  A count
  // that is not a multiple of four ends in a partial vector: the CTA whose stripe holds it
  // moves those one to three elements with scalar accesses, so nothing beyond the caller's
  // vector is read or written.
  const uint64_t vec = (p.count + 3) / 4, full = p.count / 4;
  const uint64_t v0 = min(static_cast<uint64_t>(b) * kStripeVec, vec), v1 = min(v0 + kStripeVec, vec);
  const uint64_t v1_full = min(v1, full);
  const uint32_t tail = (v0 <= full && full < v1) ? static_cast<uint32_t>(p.count - full * 4) : 0u;

  float4* my_slot = reinterpret_cast<float4*>(mine + comm_slot_off(p.slot_bytes, slot));
  const float4* src = reinterpret_cast<const float4*>(p.data);
  for (uint64_t i = v0 + threadIdx.x; i < v1_full; i += blockDim.x) my_slot[i] = src[i];
  if (threadIdx.x < tail) reinterpret_cast<float*>(my_slot)[full * 4 + threadIdx.x] = p.data[full * 4 + threadIdx.x];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.world) {
    unsigned int* flag = reinterpret_cast<unsigned int*>(p.base[threadIdx.x]) + b * kMaxWorld + p.rank;
    st_release_sys(flag, epoch);
  }
  if (threadIdx.x < p.world) {
    const unsigned int* flag = reinterpret_cast<const unsigned int*>(mine) + b * kMaxWorld + threadIdx.x;
    uint32_t spins = 0;
    // epochs only grow; signed distance handles wrap-around
    while (static_cast<int>(ld_acquire_sys(flag) - epoch) < 0) {
      if (++spins > kCommSpinLimit) {
        *reinterpret_cast<volatile int*>(p.status) = 1;
        break;
      }
    }
  }
  __syncthreads();
  float4* dst = reinterpret_cast<float4*>(p.data);
  for (uint64_t i = v0 + threadIdx.x; i < v1_full; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r = 0; r < p.world; ++r) {
      const float4 v = ld_peer_f4(reinterpret_cast<const float4*>(p.base[r] + comm_slot_off(p.slot_bytes, slot)) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    dst[i] = acc;
  }
  if (threadIdx.x < tail) {
    float acc = 0.f;
    for (uint32_t r = 0; r < p.world; ++r)
      acc += ld_peer_f32(reinterpret_cast<const float*>(p.base[r] + comm_slot_off(p.slot_bytes, slot)) + full * 4 + threadIdx.x);
    p.data[full * 4 + threadIdx.x] = acc;
  }
  if (threadIdx.x == 0) epochs[b] = epoch;
}

}  // namespace

struct Comm {
  uint32_t rank = 0, world = 0;
  uint64_t slot_bytes = 0;
  uint8_t* local = nullptr;
  uint8_t* base[kMaxWorld] = {};
  bool connected = false;
  int* status_host = nullptr;
  int* status_dev = nullptr;
  FusedCommDev* fused_dev = nullptr;  // device copy of the view, filled by comm_connect
};

Comm* comm_create(uint32_t rank, uint32_t world, uint64_t max_bytes, uint8_t* handle_out, cudaError_t* err,
                  const char** why) {
  *why = "";
  *err = cudaSuccess;
  if (max_bytes > uint64_t(kMaxBlocks) * kStripeVec * 16) {
    *why = "an exchange is at most 512 KiB";
    *err = cudaErrorInvalidValue;
    return nullptr;
  }
  if (world < 2 || world > static_cast<uint32_t>(kMaxWorld) || rank >= world) {
    *why = "world must be 2..8 and rank < world";
    *err = cudaErrorInvalidValue;
    return nullptr;
  }
  Comm* c = new Comm();
  c->rank = rank;
  c->world = world;
  c->slot_bytes = (max_bytes + 255) & ~uint64_t(255);
  const uint64_t total = fused_off(c->slot_bytes) + 256 + fused_flags_bytes() + fused_data_bytes();
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->local), total);
  if (e == cudaSuccess) e = cudaMemset(c->local, 0, total);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, c->local);
  if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&c->status_host), sizeof(int), cudaHostAllocMapped);
  if (e == cudaSuccess) {
    *c->status_host = 0;
    e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->status_dev), c->status_host, 0);
  }
  if (e != cudaSuccess) {
    *err = e;
    if (c->local) cudaFree(c->local);
    if (c->status_host) cudaFreeHost(c->status_host);
    delete c;
    return nullptr;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle_out, &h, 64);
  return c;
}

cudaError_t comm_connect(Comm* c, const uint8_t* all_handles) {
  for (uint32_t r = 0; r < c->world; ++r) {
    if (r == c->rank) {
      c->base[r] = c->local;
      continue;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, all_handles + static_cast<size_t>(r) * 64, 64);
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return e;
    c->base[r] = static_cast<uint8_t*>(ptr);
  }
  FusedCommDev view = {};
  for (uint32_t r = 0; r < c->world; ++r) view.base[r] = c->base[r];
  view.rank = c->rank;
  view.world = c->world;
  const uint64_t f0 = fused_off(c->slot_bytes);
  view.flags_off = f0 + 256;
  view.data_off = f0 + 256 + fused_flags_bytes();
  view.epoch = reinterpret_cast<unsigned int*>(c->local + f0);
  view.done = reinterpret_cast<unsigned int*>(c->local + f0 + 128);
  view.status = c->status_dev;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->fused_dev), sizeof(FusedCommDev));
  if (e == cudaSuccess) e = cudaMemcpy(c->fused_dev, &view, sizeof(view), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return e;
  c->connected = true;
  return cudaSuccess;
}

const FusedCommDev* comm_fused_view(const Comm* c) { return c && c->connected ? c->fused_dev : nullptr; }
uint32_t comm_rank(const Comm* c) { return c ? c->rank : 0; }

void comm_destroy(Comm* c) {
  if (!c) return;
  for (uint32_t r = 0; r < c->world; ++r)
    if (r != c->rank && c->base[r]) cudaIpcCloseMemHandle(c->base[r]);
  if (c->local) cudaFree(c->local);
  if (c->fused_dev) cudaFree(c->fused_dev);
  if (c->status_host) cudaFreeHost(c->status_host);
  delete c;
}

bool comm_connected(const Comm* c) { return c && c->connected; }
uint64_t comm_max_bytes(const Comm* c) { return c->slot_bytes; }

cudaError_t comm_all_reduce(Comm* c, cudaStream_t stream, float* data, uint64_t count) {
  CommParams p = {};
  for (uint32_t r = 0; r < c->world; ++r) p.base[r] = c->base[r];
  p.rank = c->rank;
  p.world = c->world;
  p.slot_bytes = c->slot_bytes;
  p.data = data;
  p.count = count;
  p.status = c->status_dev;
  // one CTA per 16 KB stripe
  const uint64_t vec = (count + 3) / 4;
  int blocks = static_cast<int>((vec + kStripeVec - 1) / kStripeVec);
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks || count * sizeof(float) > c->slot_bytes) return cudaErrorInvalidValue;
  all_reduce_kernel<<<blocks, kCommThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

int comm_take_status(Comm* c) {
  const int s = *reinterpret_cast<volatile int*>(c->status_host);
  *reinterpret_cast<volatile int*>(c->status_host) = 0;
  return s;
}

}  // namespace kq
