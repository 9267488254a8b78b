/*
 * kq.h — C ABI of libkq.so: karume's quantized `linear` op on NVIDIA B200 (sm_100a).
 *
 * karume has no native plugin interface: its backend seam is WebGPU.  The entry
 * points below stand where the TypeScript runtime issues WebGPU calls for a
 * `linear` node whose weight initializer is stored as packed int4 or int8, and each
 * one names the reference code it replaces (paths relative to the karume
 * repository).  Everything is expressible as `Deno.dlopen` symbol descriptors:
 * parameters are i32 / u32 / u64 / pointer / buffer, results are i32 status codes or
 * u64, out-values go through caller-provided pointers, there are no structs by
 * value, callbacks or varargs.
 *
 * Conventions
 *  - Every call returns a kq_status (0 = ok).  On failure the context keeps a
 *    human-readable message (kq_last_error).  Nothing falls back to another
 *    implementation: an unsupported request is an error.
 *  - Device memory is addressed by plain 64-bit device pointers (`uint64_t`); a
 *    buffer made by kq_buffer_alloc and a pointer obtained elsewhere in the same
 *    process (e.g. a framework tensor) are interchangeable.
 *  - One context = one CUDA device = one calling thread at a time (the reference
 *    serialises the runs of a Session the same way,
 *    packages/runtime/src/runtime/executor.ts:975-1008).  Calls enqueue work on the
 *    context's stream and return; kq_sync is the fence (the reference's single
 *    mapAsync fence, executor.ts:1423-1462).
 *  - Same inputs give bit-identical outputs from run to run: reductions use fixed
 *    trees and no floating-point atomics.
 */
#ifndef KQ_H_
#define KQ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KQ_API __attribute__((visibility("default")))

typedef struct kq_ctx kq_ctx;
typedef uint64_t kq_weight; /* opaque handle, 0 is never valid */
typedef uint64_t kq_graph;  /* opaque handle, 0 is never valid */
typedef uint64_t kq_plan;   /* opaque handle, 0 is never valid */

enum kq_status {
  KQ_OK = 0,
  KQ_ERR_BAD_ARG = 1,     /* null pointer, unknown enum value, stale handle */
  KQ_ERR_SHAPE = 2,       /* a shape / size predicate of the storage contract is violated */
  KQ_ERR_OOM = 3,         /* device allocation failed */
  KQ_ERR_CUDA = 4,        /* a CUDA runtime call failed; message carries the CUDA error */
  KQ_ERR_UNSUPPORTED = 5, /* valid request this build has no kernel for (never a silent alternate path) */
  KQ_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up (multi-GPU exchange) */
  /* 7 is retired (it reported activations beyond the binary16 range; the kernels now take any value) */
  KQ_ERR_STATE = 8        /* call not legal now (e.g. graph capture already open) */
};

/* storage.dtype of the weight initializer (docs/ir-v1.md:124-150, :164-186). */
enum kq_storage { KQ_STORAGE_I4 = 4, KQ_STORAGE_I8 = 8 };

/* Element types of activations, outputs and companion scales. */
enum kq_dtype { KQ_F32 = 0, KQ_F16 = 1, KQ_BF16 = 2 };

/* How a weight is cut for tensor-parallel execution (no reference counterpart:
 * karume is single-device).  COLUMN keeps rows [rank*n/world, (rank+1)*n/world) of
 * W and of the scale; ROW keeps the K range [rank*k/world, (rank+1)*k/world) of
 * every row (k/world must be a multiple of the group size) and the matching scale
 * columns. */
enum kq_shard { KQ_SHARD_NONE = 0, KQ_SHARD_COLUMN = 1, KQ_SHARD_ROW = 2 };

/* ---- context --------------------------------------------------------------
 * Replaces acquireGpu() -> GpuContext (packages/runtime/src/gpu/device.ts:1182-1218):
 * one device per context.  `device` is a CUDA ordinal.  workspace_bytes sizes the
 * context-owned scratch of the split-K kernels and the activation pre-kernels (0 = default 256 MiB). */
KQ_API int kq_init(int device, uint64_t workspace_bytes, kq_ctx** out);
KQ_API void kq_destroy(kq_ctx* ctx);

/* Message of the last failing call on this context ("" if none); with ctx == NULL
 * the message of the last failing kq_init.  The pointer stays valid until the next
 * failing call.  Mirrors the reference's typed, never-swallowed errors
 * (packages/runtime/mod.ts:13-113). */
KQ_API const char* kq_last_error(kq_ctx* ctx);

/* Work is enqueued on the context's own stream unless a foreign cudaStream_t is
 * installed here (pass 0 to return to the own stream). */
KQ_API int kq_set_stream(kq_ctx* ctx, uint64_t cuda_stream);
KQ_API int kq_sync(kq_ctx* ctx);

/* Programmatic dependent launch between consecutive kq_linear kernels (each kernel
 * prefetches its weights while its predecessor drains).  On by default. */
KQ_API int kq_set_overlap(kq_ctx* ctx, int enabled);

/* ---- device buffers ---------------------------------------------------------
 * Replace the run arena's storage buffers and queue.writeBuffer / mapAsync readback
 * (packages/runtime/src/runtime/recipe-builder.ts:409-418,
 *  packages/runtime/src/runtime/executor.ts:1423-1462). */
KQ_API int kq_buffer_alloc(kq_ctx* ctx, uint64_t bytes, uint64_t* out_dptr);
KQ_API int kq_buffer_free(kq_ctx* ctx, uint64_t dptr);
/* Asynchronous on the context's stream; the host range must stay valid until kq_sync
 * unless it is pageable memory (then the copy is staged before the call returns). */
KQ_API int kq_buffer_write(kq_ctx* ctx, uint64_t dptr, uint64_t offset, const void* host, uint64_t bytes);
KQ_API int kq_buffer_read(kq_ctx* ctx, uint64_t dptr, uint64_t offset, void* host, uint64_t bytes);
/* Page-locked host memory for the two calls above (what a Deno host would wrap in an
 * ArrayBuffer via Deno.UnsafePointerView). */
KQ_API int kq_host_alloc(kq_ctx* ctx, uint64_t bytes, void** out_host);
KQ_API int kq_host_free(kq_ctx* ctx, void* host);

/* ---- weights ------------------------------------------------------------------
 * Replaces the i4 / i8 branch of Session.#build that uploads the packed payload and
 * its companion scale once per Session
 * (packages/runtime/src/runtime/executor.ts:830-896).
 *
 * payload: the safetensors bytes of the weight, logical shape [n, k] row-major.
 *   I4: n*k/2 bytes, flat element i in byte i>>1, low nibble when i is even, stored
 *       nibble u = q + 8 (packages/runtime/src/format/i4.ts:63-118);
 *       group_size is a power of two >= 16 dividing k
 *       (packages/runtime/src/kernels/weight-storage.ts:56-70); the scale is
 *       [n, k/group_size] row-major.
 *   I8: n*k signed bytes (packages/runtime/src/format/i8.ts:80-117); group_size
 *       must be 0; the scale is [n] (the keepdim form [n,1] flattened).
 * scale_dtype: KQ_F32 is the reference's companion format; KQ_F16 is accepted as
 *   well and is widened exactly to f32 before the dequant multiply, so the
 *   dequantised weight is the same single-rounding f32 value either way.
 * payload_bytes / scale_bytes must equal the sizes the shape implies.
 * The device layout is private to the library (the bytes may be permuted for
 * coalesced streaming); no weight is ever expanded:
 * kq_weight_resident_bytes == payload_bytes + scale_bytes, the invariant the
 * reference asserts on Session.diagnostics().storage.residentCompressedBytes
 * (packages/runtime/tests/gpu_i4_weights_test.ts:170-174). */
KQ_API int kq_weight_upload(kq_ctx* ctx, int storage, const void* payload, uint64_t payload_bytes,
                            const void* scale, uint64_t scale_bytes, int scale_dtype, uint32_t n,
                            uint32_t k, uint32_t group_size, kq_weight* out);
/* Same, keeping only this rank's shard (see kq_shard).  The host passes the FULL
 * payload and scale; the shard is cut and laid out on the device. */
KQ_API int kq_weight_upload_shard(kq_ctx* ctx, int storage, const void* payload,
                                  uint64_t payload_bytes, const void* scale, uint64_t scale_bytes,
                                  int scale_dtype, uint32_t n, uint32_t k, uint32_t group_size,
                                  int shard, uint32_t rank, uint32_t world, kq_weight* out);
KQ_API int kq_weight_free(kq_ctx* ctx, kq_weight w);
KQ_API uint64_t kq_weight_resident_bytes(kq_ctx* ctx, kq_weight w);
/* Logical [n, k] of the (possibly sharded) weight held on this device. */
KQ_API int kq_weight_shape(kq_ctx* ctx, kq_weight w, uint32_t* out_n, uint32_t* out_k);

/* Expands the resident weight to f32 [n, k] row-major with the kernels' own dequant
 * rule.  Replaces the load-time CPU expansion of ineligible initializers
 * (decodeI4 / decodeI8, executor.ts:851, :887) and is what the bit-exactness tests
 * read (packages/runtime/tests/gpu_i4_weights_test.ts:404-459,
 *       packages/runtime/tests/gpu_i8_weights_test.ts:612-660). */
KQ_API int kq_weight_dequant(kq_ctx* ctx, kq_weight w, uint64_t out_f32_dptr);

/* ---- models in karume's distribution format ----------------------------------------------
 * A model is ONE .safetensors file (8-byte little-endian header length, header JSON, data
 * section) whose __metadata__.karume_ir holds the graph JSON (docs/ir-v1.md).  kq_model_open
 * reads it with the reference's own checks and refuses what the reference refuses:
 *   - header: known dtypes, integer shapes, byte size == numel * bits / 8 (I4 = 4 bits; an odd
 *     number of I4 elements is refused), the data section covered exactly (no overlap, gap or
 *     tail), every tensor start aligned (I4: 4 bytes)
 *     (packages/runtime/src/format/safetensors.ts:25-50, :107-160, :187-262);
 *   - initializers: storage { dtype, scale, group_size } with scale required for i8 / i4,
 *     group_size required for i4 (a power of two >= 16 dividing numel / shape[0]) and refused
 *     on any other storage (packages/runtime/src/format/ir.ts:268-306, :617-646;
 *     packages/runtime/src/format/container.ts:468-506);
 *   - against the file: tensor present, dtype == the storage's encoding, shape == the declared
 *     one; scale tensors F32, [shape[0], row / group_size] for i4 and the keepdim broadcast form
 *     for i8; no tensor without a referring initializer
 *     (packages/runtime/src/format/container.ts:180-232, :309-320, :337-400).
 * The graph's nodes stay the host's business.  These calls need no GPU and no context; their
 * error text is read with kq_last_error(NULL).  kq_model_weight uploads one packed i4 / i8
 * initializer (rank >= 2, rows = shape[0], k = numel / shape[0]) as a resident weight. */
typedef uint64_t kq_model; /* opaque handle, 0 is never valid */
KQ_API int kq_model_open(const char* path, kq_model* out);
KQ_API int kq_model_open_memory(const void* bytes, uint64_t size, kq_model* out); /* the bytes are copied */
KQ_API void kq_model_close(kq_model model);
KQ_API uint32_t kq_model_initializer_count(kq_model model);
KQ_API const char* kq_model_initializer_name(kq_model model, uint32_t index);
/* Any out-pointer may be NULL.  storage_bits: 4 (i4), 8 (i8), 16 (f16 / bf16), 32 (f32 / i32);
 * shape8 receives up to 8 dimensions (the rest 0); payload / scale point into the model's copy
 * of the file and stay valid until kq_model_close. */
KQ_API int kq_model_initializer_info(kq_model model, const char* name, uint32_t* storage_bits, uint32_t* rank,
                                     uint64_t* shape8, uint32_t* group_size, const void** payload,
                                     uint64_t* payload_bytes, const void** scale, uint64_t* scale_bytes);
KQ_API int kq_model_weight(kq_ctx* ctx, kq_model model, const char* name, kq_weight* out);
/* A .safetensors file without a graph (the reference's golden io files): the header checks
 * only.  kq_model_tensor_info looks a tensor up by its safetensors key in either kind of
 * handle; dtype8 receives the dtype name ("F32", "I8", "I4", ...), NUL-terminated. */
KQ_API int kq_tensors_open(const char* path, kq_model* out);
KQ_API int kq_model_tensor_info(kq_model model, const char* key, char* dtype8, uint32_t* rank, uint64_t* shape8,
                                const void** data, uint64_t* bytes);

/* ---- the op ---------------------------------------------------------------------
 * out[m, n] = sum_k x[m, k] * W[n, k] + bias[n], f32 accumulate, f32 output.
 * Replaces RecipeBuilder.#buildLinear's pipeline lookup + dispatch
 * (packages/runtime/src/runtime/recipe-builder.ts:1311-1392; bindings 1 x, 2 w,
 * 3 bias, 4 out, 5 wscale — packages/runtime/src/kernels/gemm.ts:1223-1227).
 * x is [m, k] row-major of x_dtype (leading dims flattened by the caller, as
 * #buildLinear does); bias is f32 [n] and always present (arity 3 is fixed,
 * packages/runtime/src/ops/shapes.ts:502-523); out is f32 [m, n].
 * The kernel is a pure function of (storage, shape, m, x_dtype) — never autotuned,
 * like the reference's geometry table
 * (packages/runtime/src/kernels/gemm-geometry.ts:243-267).
 * More than 16 rows on a tiled int4 weight run on the tcgen05 tensor cores: bf16 activations
 * with operands rounded to bf16 once (results within rtol 1e-3, atol 1e-4 * rms of the oracle
 * on bf16-rounded operands), f32 / binary16 activations with both operands carried as two bf16
 * numbers (the decode contract, atol 4e-5 * max(1, rms) for f32 activations).  A tiled int8
 * weight with k % 64 == 0 takes the same bf16 kernel and contract; its other cases, and
 * everything up to 16 rows, keep atol 1e-5 * max(1, rms), rtol 1e-3 against the f64-accumulate
 * reference. */
KQ_API int kq_linear(kq_ctx* ctx, kq_weight w, uint64_t x_dptr, int x_dtype, uint64_t bias_dptr,
                     uint64_t out_dptr, uint32_t m);

/* Several weights applied to the SAME x in one launch (q/k/v, gate/up).  Outputs
 * are separate [m, n_i] tensors; semantics are those of `count` kq_linear calls. */
KQ_API int kq_linear_multi(kq_ctx* ctx, uint32_t count, const kq_weight* w, uint64_t x_dptr,
                           int x_dtype, const uint64_t* bias_dptr, const uint64_t* out_dptr,
                           uint32_t m);

/* Host-buffer form of kq_linear: copies x in, runs, copies out, and returns after
 * the result is in `out_host` (the round trip Session.run makes per call,
 * executor.ts:985-1507).  bias stays a device pointer: it is a weight-lifetime
 * initializer. */
KQ_API int kq_linear_host(kq_ctx* ctx, kq_weight w, const void* x_host, int x_dtype,
                          uint64_t bias_dptr, float* out_host, uint32_t m);

/* One linear for callers that must not allocate device memory (no counterpart in the
 * reference, whose WebGPU layer always allocates through its arena).  Some hosts cannot
 * afford a cudaMalloc on the inference path: a serving process that has handed all free
 * HBM to its own cache pool (an allocation then fails or fragments that pool), or a loop
 * with a latency budget that cudaMalloc's implicit device-wide synchronisation would
 * break.  This call computes the same out = x . W^T + bias as kq_linear for an int4 /
 * group-32 weight in the tiled layout and m <= 16 with the fused plan kernel, and takes
 * the global scratch that kernel needs (barrier word, status word, op descriptor) from one
 * static 4 KiB array inside the library, which each GPU holds from the moment it loads
 * libkq until the process exits.  Neither this call nor anything it calls uses cudaMalloc,
 * cudaFree or an allocating library routine.
 *  - Limit: the op's activations are staged whole in shared memory, so k * c * 2 bytes
 *    (c = m for binary16 activations, 2 m for f32 / bf16) plus the weight rings must fit
 *    227 KiB: e.g. k <= 14336 at m = 1 in f32, k <= 4096 at m = 8.  Beyond that the call
 *    returns KQ_ERR_UNSUPPORTED and runs nothing.
 *  - The first call on a device looks up the array's device address and zeroes it; make
 *    that first call outside any stream capture.
 *  - All calls share the one array, which keeps the previous call's contents; the words
 *    that must start at zero are cleared by every call.  Two calls whose kernels overlap
 *    on the GPU (different streams or contexts of one device) race on it, so the call
 *    returns only after its kernel has finished and must not be issued concurrently.
 *  - Weight, x, bias and out are the caller's, exactly as for kq_linear. */
/* The same linear (one to four weights on one x, as kq_linear_multi) on the tcgen05 tensor
 * cores: the weights are the 128-row side of the MMA, written into tensor memory straight from
 * the packed layout, the activations its 16 columns, one f32 accumulator per scale group.
 * Covered: tiled int4 / group-32 weights of one k and scale type, 5..16 binary16 rows or 5..8
 * f32 / bf16 rows, k % 64 == 0; anything else returns KQ_ERR_UNSUPPORTED.  Same results contract
 * as kq_linear.  kq_linear does not route here: on B200 the mma.sync kernels it uses are faster
 * for these shapes (an MMA of 16 columns costs the tensor core as much as one of 64, and tensor
 * memory bounds how many 64-k steps can be in flight); the entry point exists so that a host can
 * choose and measure.  Uses the context's scratch; cannot be recorded into a fused plan. */
KQ_API int kq_linear_tc(kq_ctx* ctx, uint32_t count, const kq_weight* w, uint64_t x_dptr, int x_dtype,
                        const uint64_t* bias_dptr, const uint64_t* out_dptr, uint32_t m);

KQ_API int kq_linear_static(kq_ctx* ctx, kq_weight w, uint64_t x_dptr, int x_dtype, uint64_t bias_dptr,
                            uint64_t out_dptr, uint32_t m);

/* ---- the matmul's neighbours in a decoder layer -------------------------------------------
 * rms_norm, the SiLU gate and the residual add are separate kernels in the reference
 * (packages/runtime/src/kernels/rms-norm.ts, packages/runtime/src/kernels/silu.ts fused from
 * sigmoid -> mul by packages/runtime/src/runtime/fusion.ts:453-511, and the elementwise `mul` /
 * `add`).  They are exported here with the reference's f32 formulas:
 *   kq_rms_norm  out[r, i] = x[r, i] * rsqrt(mean_r(x^2) + eps) * weight[i]   (eps > 0, inside the root)
 *   kq_silu_mul  out[i] = (gate[i] * sigmoid(gate[i])) * up[i], sigmoid(x) = t = exp(-|x|); x < 0 ? t/(1+t) : 1/(1+t)
 *   kq_add       out[i] = a[i] + b[i]
 * All tensors f32; out may alias an input of kq_silu_mul / kq_add. */
KQ_API int kq_rms_norm(kq_ctx* ctx, uint64_t x_dptr, uint64_t weight_dptr, float eps, uint64_t out_dptr, uint32_t rows,
                       uint32_t dim);
KQ_API int kq_silu_mul(kq_ctx* ctx, uint64_t gate_dptr, uint64_t up_dptr, uint64_t out_dptr, uint64_t count);
KQ_API int kq_add(kq_ctx* ctx, uint64_t a_dptr, uint64_t b_dptr, uint64_t out_dptr, uint64_t count);

/* kq_linear_fused: a linear with those neighbours attached, the four shapes a decoder layer
 * is made of.  The result is that of the node sequence
 *   [rms_norm(x, norm_weight, eps) ->] linear(s) [-> silu(gate) * up] [-> all-reduce over ranks] [-> + residual]
 * with every node's output rounded to f32 as the reference rounds it.
 *   norm_weight_dptr  0, or f32 [k]: x (f32) is normalised first
 *   flags & KQ_FUSE_SWIGLU  count == 2, weights (gate, up) of equal shape: ONE output
 *                     out_dptr[0][m, n] = silu(x.Wg^T + bias[0]) * (x.Wu^T + bias[1])
 *   flags & KQ_FUSE_REDUCE  count == 1: the weight is a KQ_SHARD_ROW shard, x its k slice; the
 *                     outputs are added across the connected ranks (as kq_linear_reduce), then
 *                     the bias and the residual are added, the same bits on every rank
 *   residual_dptr     0, or f32 [m, n] (count == 1); may be the same buffer as out_dptr[0]
 * out must not alias x.  Called directly it runs as separate kernels (norm, linears, gate or
 * add).  Recorded into a fused plan (kq_plan_begin .. kq_plan_end) the persistent kernel does
 * the norm while it stages the activations and the gate / exchange / residual in the epilogue
 * of the matmul, so gate and up never travel through HBM; that needs the plan's paired kernel
 * (at most two f32 / bf16 rows or four binary16 rows, n a multiple of 32 except for the gate
 * pair, at most 8192 outputs per exchanged op), else kq_plan_end returns KQ_ERR_UNSUPPORTED. */
enum kq_fuse { KQ_FUSE_SWIGLU = 1, KQ_FUSE_REDUCE = 2 };
KQ_API int kq_linear_fused(kq_ctx* ctx, uint32_t count, const kq_weight* w, uint64_t x_dptr, int x_dtype,
                           uint64_t norm_weight_dptr, float norm_eps, const uint64_t* bias_dptr,
                           uint64_t residual_dptr, const uint64_t* out_dptr, uint32_t m, uint32_t flags);

/* ---- embedding gather ----------------------------------------------------------------
 * out[row, :] = dequantised row index[row] of a resident weight [vocab, hidden] (the weight a
 * tied LM head shares), f32.  Replaces the packed-weight variants of the reference's embedding
 * kernel (packages/runtime/src/kernels/embedding.ts:70-117): same single-multiply dequant as
 * kq_weight_dequant, and an index outside [0, vocab) writes quiet NaNs into its row instead
 * of returning another row.  index is int32 [rows]. */
KQ_API int kq_embedding(kq_ctx* ctx, kq_weight w, uint64_t index_i32_dptr, uint32_t rows, uint64_t out_dptr);

/* ---- integer-dot form (w8a8 / w4a8) ------------------------------------------------
 * kq_quantize_rows replaces the reference's activation quantiser
 * (packages/runtime/src/kernels/quantize-rows.ts:83-155): per row of x[rows, dim] (f32),
 *   scale[row] = max(max|x| * (1/127), f32 tiny)   (NaN in the row -> NaN scale)
 *   q[row, i]  = clamp(round_ties_even(x / scale), -127, 127) as int8, correctly rounded division.
 * kq_linear_a8 replaces the integer GEMM variants (packages/runtime/src/kernels/linear-i8a8.ts:21-72,
 * stated on the CPU by packages/runtime/src/reference/i8a8.ts:159-229), chosen by the
 * weight's storage:
 *   int8: out = fma(f32(sum_k xq * wq), fround(xs[row] * ws[col]), bias[col]),  k <= 131072
 *   int4: accf = fma(f32(sum_{k in group} xq * wq), ws[col, group], accf), groups ascending;
 *         out = fma(accf, xs[row], bias[col])
 * Integer sums are exact, so results are bit-identical to the reference's CPU statement
 * (its own tests compare with atol = 0).  xq is int8 [m, k] row-major, xs f32 [m]. */
KQ_API int kq_quantize_rows(kq_ctx* ctx, uint64_t x_f32_dptr, uint32_t rows, uint32_t dim, uint64_t q_i8_dptr,
                            uint64_t scale_f32_dptr);
KQ_API int kq_linear_a8(kq_ctx* ctx, kq_weight w, uint64_t xq_i8_dptr, uint64_t xs_f32_dptr, uint64_t bias_dptr,
                        uint64_t out_dptr, uint32_t m);

/* ---- replayable plans -----------------------------------------------------------
 * Records every kq_* launch between begin and end into a CUDA graph that
 * kq_graph_launch replays.  Replaces the reference's baked plan replay
 * (executeBakedPlan, packages/runtime/src/runtime/recipe.ts:462). */
KQ_API int kq_graph_begin(kq_ctx* ctx);
KQ_API int kq_graph_end(kq_ctx* ctx, kq_graph* out);
KQ_API int kq_graph_launch(kq_ctx* ctx, kq_graph g);
KQ_API int kq_graph_free(kq_ctx* ctx, kq_graph g);

/* ---- fused plans ----------------------------------------------------------------
 * Same role as kq_graph_* (the reference's baked-plan replay, recipe.ts:462), different
 * execution: between begin and end, kq_linear / kq_linear_multi / kq_buffer_write /
 * kq_buffer_read are RECORDED, not run; kq_plan_launch then executes all recorded linears
 * inside one persistent kernel that keeps streaming weights across the dependencies
 * between them, with the recorded host->device copies before it and the device->host
 * copies after it.  Ops run in recording order and each one sees the outputs of all
 * earlier ones.  Covered: int4 / group-32 weights in the library's tiled layout
 * (n % 16 == 0, k % 64 == 0), one activation type, one m <= 16 and one scale type for the
 * whole plan, and the widest op's activations (k * columns * 2 bytes) must fit in shared
 * memory next to the weight rings; anything else makes kq_plan_end return
 * KQ_ERR_UNSUPPORTED (record such a sequence with kq_graph_begin instead).  A bounded
 * device-side wait that gives up is reported by the next kq_sync as KQ_ERR_TIMEOUT. */
KQ_API int kq_plan_begin(kq_ctx* ctx);
KQ_API int kq_plan_end(kq_ctx* ctx, kq_plan* out);
KQ_API int kq_plan_launch(kq_ctx* ctx, kq_plan plan);
KQ_API int kq_plan_free(kq_ctx* ctx, kq_plan plan);
/* Runs the plan once (copies included) with phase stamps switched on and returns them: the
 * fused kernel's counterpart of the reference's per-pipeline timestamp queries
 * (packages/runtime/src/gpu/submit.ts:180-194, docs/decisions/0021-gpu-timing-diagnostics.md).
 * stamps[(cta * ops + op) * slots + s] is the GPU's nanosecond timer when CTA `cta` reached point
 * s of op `op`: 0 done with the previous op, 1 through the grid barrier, 2 activations staged,
 * 3 first weight piece landed (warp 0), 4 weights of the first round consumed (warp 0), 5 outputs
 * stored; the other slots are zero.  With stamps == NULL only the three sizes are returned.
 * Plans that run on the paired kernel only (at most two f32 rows); allocates and frees its
 * buffer, so not for the serving path. */
KQ_API int kq_plan_profile(kq_ctx* ctx, kq_plan plan, uint64_t* stamps, uint64_t capacity, uint32_t* out_ctas,
                           uint32_t* out_ops, uint32_t* out_slots);

/* ---- tensor-parallel exchange --------------------------------------------------------
 * No reference counterpart (karume is single-device).  One process per GPU: every rank
 * calls kq_comm_create (allocates its exchange buffer and returns a 64-byte IPC handle),
 * the host gathers the handles of all ranks in rank order by any means, and every rank
 * passes the concatenation (world * 64 bytes) to kq_comm_connect.  kq_all_reduce then sums
 * an f32 vector of up to max_bytes (<= 512 KiB) over the ranks in place, with one kernel
 * that reads the peers' buffers over NVLink; the sum is taken in rank order, so all ranks
 * hold the same bits.  Every rank must issue the same sequence of kq_all_reduce calls.
 * The kernel can be captured in a CUDA graph.  A peer that does not arrive within the
 * kernel's bounded wait is reported by the next kq_sync as KQ_ERR_TIMEOUT (the context stays
 * usable; a rank that was late can still make the same call and catches up).
 * Teardown: kq_destroy unmaps the peers' buffers and frees the exported one.  All ranks must
 * have finished their last exchange (kq_sync) and met at a host-side barrier before any of
 * them calls kq_destroy, so that no peer's kernel still reads or writes the freed buffer. */
KQ_API int kq_comm_create(kq_ctx* ctx, uint32_t rank, uint32_t world, uint64_t max_bytes, uint8_t* out_handle);
KQ_API int kq_comm_connect(kq_ctx* ctx, const uint8_t* all_handles);
KQ_API int kq_all_reduce(kq_ctx* ctx, uint64_t f32_dptr, uint64_t count);
/* Row-parallel linear: out = sum over ranks of (x_r . W_r^T) + bias, the same bits on every rank;
 * every rank passes its K shard of W (KQ_SHARD_ROW) and the matching slice of x.  For the decode
 * shapes (tiled int4 weight, one or two f32 / bf16 rows or up to four binary16 rows, a grid that
 * is resident in one wave) this is ONE kernel: each CTA of the GEMV pushes its partial sums into
 * the peers' exchange areas over NVLink, raises a flag there, waits (bounded) for the same CTA of
 * every peer and adds the ranks' values in rank order.  Otherwise it runs kq_linear (bias on rank 0
 * only) followed by kq_all_reduce.  All ranks must issue the same sequence of calls. */
KQ_API int kq_linear_reduce(kq_ctx* ctx, kq_weight w, uint64_t x_dptr, int x_dtype, uint64_t bias_dptr,
                            uint64_t out_dptr, uint32_t m);

/* ---- timing ---------------------------------------------------------------------
 * CUDA events on the context's stream.  Replaces the reference's opt-in
 * timestamp-query diagnostics (packages/runtime/src/gpu/submit.ts:180-194). */
KQ_API int kq_timer_start(kq_ctx* ctx);
KQ_API int kq_timer_stop(kq_ctx* ctx, float* out_ms); /* synchronises */

/* Number of kernels this library has launched on the context so far. */
KQ_API uint64_t kq_launch_count(kq_ctx* ctx);

/* Library / build identification: "kq <version> sm_100a". */
KQ_API const char* kq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KQ_H_ */
