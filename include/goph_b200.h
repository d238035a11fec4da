/* goph_b200.h — C ABI of libgoph_b200.so: B200 (sm_100a) kernels for the quantized
 * matrix-product path of rcarmo/go-pherence.
 *
 * The library replaces the PTX modules that the reference loads at run time in
 * backends/nvidia/runtime and the driver calls around them.  Every entry point takes
 * plain integers, floats and pointers so that the reference's FFI (purego, no cgo) can
 * bind it directly; the Go-side operator signatures stay as they are.  Each declaration
 * cites the reference interface it stands behind (file:line inside the reference
 * repository).
 *
 * Conventions
 *   - Return value: 0 on success, otherwise a GOPH_E_* code; goph_last_error() gives the
 *     text (with the CUDA error name when there is one).  Nothing throws, nothing aborts.
 *   - Malformed arguments are rejected before any allocation or launch, as the reference
 *     does (backends/nvidia/runtime/mlx.go:34-55, :231-249).
 *   - There is NO CPU fallback: where the reference's DevBuf operators silently run the
 *     CPU implementation on failure (mlx.go:322-349) this library returns an error.
 *   - Pointers named *_dev are device addresses on the handle's GPU; all others are host.
 *   - `stream` is a cudaStream_t / CUstream passed as void*; NULL is the legacy default
 *     stream, which is what the reference launches on (runtime.go:676).
 *   - Calls may come from any OS thread; the library sets the device it needs on every
 *     call and keeps no thread-local state besides the error text.  Like the reference
 *     (global cudaMu, runtime.go:134-139) callers serialise calls that share a handle.
 *   - The tensor-core products (tiled layouts), the attention kernel and the argmax kernel keep
 *     one scratch area per device (activation digits, split-K partial sums, counters).  Calls
 *     on one device whose kernels could overlap on the GPU — different streams with no ordering
 *     between them — must be ordered by the caller (one stream, or events), whatever handles
 *     they use.  The reference launches everything on one stream, which satisfies this.
 *   - Matrices are row-major; x is [batch, in_dim], out is [batch, out_dim], both f32.
 */
#ifndef GOPH_B200_H
#define GOPH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  GOPH_OK = 0,
  GOPH_E_INVALID = 1, /* malformed argument (nil, short buffer, bad dims, overflow) */
  GOPH_E_CUDA = 2,    /* a CUDA call failed; text carries the cudaError name */
  GOPH_E_NOINIT = 3,  /* goph_init was not called for this device */
  GOPH_E_UNSUPPORTED = 4,
  GOPH_E_NOMEM = 5
};

/* GGUF tensor type ids accepted by goph_gguf_upload (loader/gguf/gguf.go:51-56).  Q5_K and Q6_K
   (176- and 210-byte super-blocks of 256 elements; loader/gguf/quant_matrix.go:331-426) go through
   the CUDA-core streaming kernel at file size, or, for large matrices ("gguf_layout"), to the
   tensor-core kernel with their values written out as one byte per weight. */
enum { GOPH_GGUF_Q8_0 = 8, GOPH_GGUF_Q4_K = 12, GOPH_GGUF_Q5_K = 13, GOPH_GGUF_Q6_K = 14 };

typedef struct goph_mlx_weight goph_mlx_weight;   /* nvidia.GPUMLXWeight      (runtime/mlx.go:21-32)   */
typedef struct goph_gguf_matrix goph_gguf_matrix; /* nvidia.GPUGGUFMatrix / GPUQ4KMatrix / GPUQ8_0Matrix
                                                     (runtime/gguf_matrix.go:11-17, q4k.go:39-47, q8.go:20-25) */
typedef struct goph_gather goph_gather;           /* exchange area of one rank for row-sharded outputs; no counterpart
                                                     in the reference, which runs on one GPU (model/gpu_forward.go) */
typedef struct goph_moe_layer goph_moe_layer;     /* the MoE fields of model.LlamaLayer: RouterW, ExpertGateW/UpW/DownW
                                                     (model/moe.go:24-60) with their GPU copies (model/moe_gpu.go:60-110) */
typedef struct goph_fp8_linear goph_fp8_linear;   /* nvidia.GPUFP8E4M3Linear  (runtime/fp8.go:35-44)   */

/* ---- runtime: replaces Init/EnsureContext/Malloc/Upload/Download/Sync -------------- */

/* nvidia.Init + EnsureContext (runtime/runtime.go:142-274): bind `device`, create the
 * primary context, read the SM count.  Idempotent per device. */
int goph_init(int device);
/* nvidia.EnsureContext for a caller that owns its driver context, as the reference does: it creates
 * one with cuCtxCreate and allocates every buffer in it (runtime/runtime.go:226-274).  Call this
 * with that context current on the thread, INSTEAD of goph_init: the library then makes that context
 * current at the top of every entry point (calls may come from any OS thread, runtime.go:258-274),
 * launches its kernels in it, allocates its own scratch in it, and leaves it current on return, so
 * buffers from the caller's cuMemAlloc are valid arguments.  *out_device receives the device
 * ordinal of the context, which is the `device` argument of the other entry points.  A device
 * serves one context per process: mixing goph_init and this call on one device is refused. */
int goph_init_current_context(int* out_device);
/* Text of the last error on the calling thread ("" if none). */
const char* goph_last_error(void);
/* nvidia.SMCount (runtime/runtime.go:285); 0 if the device is not initialised. */
int goph_sm_count(int device);

/* Tuning switches.  The reference reads its own from GO_PHERENCE_* environment variables at
 * the call sites (model/gpu_forward.go:24-47, :776-785); here they are set by name:
 *   "pdl"         1 (default) launches kernels with programmatic stream serialization so a kernel's
 *                 prologue and weight prefetch overlap the tail of the kernel in front; 0 plain launches
 *   "mlx_layout"  device layout chosen by goph_mlx_upload.  The tiled layout feeds the tensor-core
 *                 (tcgen05) kernel and needs group size 64, in_dim a multiple of 256 and bf16-valued
 *                 scales and biases; the row-major layout feeds the CUDA-core kernels.  0 (default):
 *                 tiled for matrices of 8 Mi weights or more, row-major below; 1: always row-major;
 *                 2: tiled whenever the shape allows
 *   "gguf_layout" the same choice for goph_gguf_upload (Q4_K, Q5_K, Q6_K, Q8_0; in_dim a multiple of 256;
 *                 Q5_K and Q6_K take 1.06 / 1.13 bytes per weight in the tensor-core layout):
 *                 0 (default) tensor-core layout from 8 Mi weights, 1 always the streaming layout,
 *                 2 tensor-core layout whenever the shape allows.  "mlx_digits" and "mlx_splits"
 *                 apply to these products as well
 *   "fp8_layout"  the same choice for goph_fp8_upload (in_dim a multiple of 256, no NaN codes in the
 *                 weight): the tensor-core layout serves every batch size on the tensor cores (the
 *                 e4m3 bytes go to the MMA as they lie; f32 activations as six e4m3 pieces, exact,
 *                 bf16 activations as two); the row-major layout is served by the CUDA-core kernels
 *   "fp8_convert" 1: bf16 batches of more than 32 rows on a tensor-core FP8 linear go through the
 *                 kernel that turns the e4m3 bytes into bf16 (ahead at 8192 x 8192 x 64, behind on
 *                 matrices with more row tiles); 0 (default): the e4m3 kernel serves every batch
 *   "mlx_digits"  signed base-128 digits each activation is written in on the tensor-core path,
 *                 relative to the largest magnitude of its 64-element group: 4 (default, 27 bits)
 *                 or 3 (20 bits; enough for bf16-valued activations)
 *   "mlx_fuse"    1 (default): tensor-core launches of one or two activation rows make the activation
 *                 digits of their own K range inside the product kernel (one launch per product);
 *                 0: a separate preparation kernel in front of every product
 *   "mlx_chunks"  256-element chunks per pipeline stage of the tensor-core GEMV: 0 (default) two for
 *                 the nibble formats where tensor memory has the columns (up to 4 activation rows
 *                 for MLX 4-bit, 2 for Q4_K), 1 always one
 *   "mlx_splits"  CTAs that share the K range of one 128-row tile (0 = chosen by shape)
 *   "mlx_cluster" 1 (default): K splits that all run at once are launched as thread-block clusters and
 *                 add their partial sums through shared memory; 0: always through device scratch
 *                 and an atomic counter.  Same bits either way
 *   "moe_fused"   1 (default): an MoE call of one token on row-major experts runs as ONE cooperative
 *                 launch (router, routing, gate|up, down and the weighted sum as phases between
 *                 grid-wide barriers), and with more tokens the router rows and the routing share a
 *                 launch; 0: one launch per step of the call, for any number of tokens.  Same bits.
 *                 A barrier wait that gives up (about a second) sets the kernel status to 700 + the
 *                 barrier's number; the layer's later one-launch calls then return without
 *                 computing until goph_kernel_status_clear has been called
 *   "moe_rows"    MoE layers whose experts are in the tiled layout: (token, slot) items per work
 *                 entry of the grouped tensor-core launches, 2 or 4; 0 (default) = two while the
 *                 call has fewer than two items per expert on average, else four.  Same bits either way
 *   "mlx_unpack"  nibble→f32 method of the batch-1 MLX kernel: 0 one shift per nibble,
 *                 (default), 1 one shift per nibble pair, 2 integer conversion
 *   "mlx_rows" / "gguf_rows" / "fp8_rows"  rows a warp streams at once: 1, 2, 4, or 0 = by size
 * Unknown names and values out of range are rejected.  Results stay within the product
 * tolerance for every setting. */
int goph_set_option(const char* name, int value);
/* Device-side health word.  Every wait inside a kernel is bounded; a wait that gives up
 * stores a non-zero code here and the kernel winds down instead of hanging.  0 = no wait
 * has ever given up on this device.  (The reference localises device faults by synchronising
 * after every launch under GO_PHERENCE_CUDA_LAUNCH_CHECK, runtime/runtime.go:687-694.)
 * Synchronises with the device. */
int goph_kernel_status(int device, int* out_status);
/* Sets the device's status words back to 0 after the caller has dealt with a non-zero status
 * (the reference has no counterpart: it tears the context down).  Synchronises with the device. */
int goph_kernel_status_clear(int device);
/* No counterpart in the reference.  Number of compute kernels this process has launched through the
 * library so far (products, their activation preparation, exchanges, decode-step operations; not
 * the kernels of uploads and dequantisation).  A benchmark reads it before and after one step made
 * of plain launches to know how many kernels a step is; launches replayed by a CUDA graph are
 * counted when they are captured, not when the graph runs. */
int goph_launch_count(uint64_t* out_count);
/* nvidia.Malloc / MallocBytes / Buffer.Free (runtime/runtime.go:297-359, q8.go:166-177). */
int goph_malloc(int device, uint64_t bytes, void** out_dev);
int goph_free(int device, void* dev);
/* Buffer.Upload / UploadBytes / UploadUint32 / Download (runtime/runtime.go:382-525):
 * synchronous copies. */
int goph_upload(int device, void* dst_dev, const void* src_host, uint64_t bytes);
int goph_download(int device, void* dst_host, const void* src_dev, uint64_t bytes);
int goph_memset(int device, void* dst_dev, int byte, uint64_t bytes);
/* nvidia.Sync / SyncErr (runtime/runtime.go:551-577). */
int goph_sync(int device);

/* ---- MLX 4-bit affine weights (backends/mlx, backends/nvidia/runtime/mlx.go) -------- */

/* nvidia.UploadMLXWeight / UploadMLXWeightNative (runtime/mlx.go:59, :189).
 * weight: [out_dim, in_dim/8] uint32, element e of a word in bits 4e..4e+3;
 * scales, biases: [out_dim, in_dim/group_size] f32.  *_len are element counts of the
 * caller's slices (validated like validateMLXUploadInputs, mlx.go:34-55).
 * Scales and biases are kept as bf16 on the device when every value is exactly
 * representable in bf16 (checkpoints store them so; backends/mlx/load.go:148-157 widens
 * them), otherwise as f32; either way the arithmetic uses the exact f32 values. */
int goph_mlx_upload(int device, const uint32_t* weight, uint64_t weight_len, const float* scales,
                    const float* biases, uint64_t scale_len, int in_dim, int out_dim,
                    int group_size, goph_mlx_weight** out);
/* Same, from buffers already on the device (no host copy). */
int goph_mlx_upload_dev(int device, const uint32_t* weight_dev, const float* scales_dev,
                        const float* biases_dev, int in_dim, int out_dim, int group_size,
                        goph_mlx_weight** out);
/* GPUMLXWeight.Free (runtime/mlx.go:252-275); NULL is accepted. */
int goph_mlx_free(goph_mlx_weight* w);
/* Bytes the weight occupies on the device (packed words + scale/bias table). */
uint64_t goph_mlx_resident_bytes(const goph_mlx_weight* w);
/* mlx.DequantTo on the device (backends/mlx/dequant.go:30-42): out_dev [out_dim,in_dim]
 * f32, bit-identical to float32(nibble)*scale + bias with two roundings. */
int goph_mlx_dequant(const goph_mlx_weight* w, float* out_dev, uint64_t out_len, void* stream);
/* nvidia.GemvMLX / GemvMLXDirect (runtime/mlx.go:287-350, :455-488): out = W·x. */
int goph_mlx_gemv(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                  const goph_mlx_weight* w, void* stream);
/* nvidia.GemmMLX (runtime/mlx.go:395-431): x [batch,in] → out [batch,out].  Tiled weights: up to
 * 8 rows run on the integer tensor-core kernel; more rows on the bf16 tensor-core kernel, which
 * streams the weights once per 16 rows (every f32 activation is split into three bf16 pieces
 * that add up to it exactly, so the result is as exact as the 8-row path's). */
int goph_mlx_gemm(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                  const goph_mlx_weight* w, int batch, void* stream);
/* nvidia.GemmMLX (runtime/mlx.go:395-431) for activations held as bf16 (prefill chunks and verifier
 * batches of models whose activations are bf16): x_bf16_dev is [batch,in] bf16 bit patterns,
 * 16-byte aligned; x_len counts elements.  The weights are streamed once per 64 rows.  Tiled
 * weights only (GOPH_E_UNSUPPORTED otherwise). */
int goph_mlx_gemm_bf16(float* out_dev, uint64_t out_len, const uint16_t* x_bf16_dev, uint64_t x_len,
                       const goph_mlx_weight* w, int batch, void* stream);
/* mlx.Gemv2To generalised (backends/mlx/gemv.go:32-60): n ≤ 8 weights with equal in_dim and
 * group size share one x [batch,in]; outs_dev[i] is [batch, out_dim_i].  One launch. */
int goph_mlx_gemm_multi(int n, float* const* outs_dev, const goph_mlx_weight* const* ws,
                        const float* x_dev, uint64_t x_len, int batch, void* stream);
/* No counterpart in the reference.  out = W·x (batch 1) for a weight in the tiled layout, computed
 * without allocating: no cudaMalloc, cudaFree or allocating library call happens inside.  It is
 * meant for callers that cannot allocate device memory at the point where they need a product —
 * a serving loop whose memory budget is fully committed to KV and expert pools, a thread that must
 * not take the allocator's device-wide synchronisation in the middle of a decode step, or code that
 * is already capturing its stream.  The kernel's scratch (health word, tile counters, prepared
 * activation digits, split-K partial sums) lives in a 242 KiB array that is part of the library
 * image on every GPU that loads it.
 * Limits: in_dim <= 16384, out_dim <= 524288, batch 1, tiled layout only (group size 64, in_dim a
 * multiple of 256, bf16-valued scales/biases, uploaded with "mlx_layout" 0 or 2) — anything else
 * is rejected with GOPH_E_UNSUPPORTED and a text that names the limit.  x_dev must be 16-byte aligned.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress) and makes
 * the driver load the kernels it launches; make that first call before any stream capture begins.
 * All calls on a device share the one array: calls that can overlap on the GPU (different streams
 * without an ordering between them) race on it, so keep them in one stream or order them with
 * events.  The array keeps the previous call's contents; the entry point clears the tile counters,
 * which must start at zero, with a memset on `stream`.  Its health word (see goph_kernel_status) is
 * part of the array, sticky, and read with goph_mlx_gemv_noalloc_status, which allocates nothing. */
int goph_mlx_gemv_noalloc(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                          const goph_mlx_weight* w, void* stream);
/* No counterpart in the reference.  0, or the code of the first bounded wait that gave up inside a
 * goph_mlx_gemv_noalloc kernel on this device.  Synchronises with the device; allocates nothing. */
int goph_mlx_gemv_noalloc_status(int device, int* out_status);
/* Host-slice form, as nvidia.GemvQ4K/GemmFP8E4M3 take Go slices (runtime/q4k.go:571,
 * fp8.go:180): copies x in, runs, copies out back, synchronises. */
int goph_mlx_gemm_host(float* out_host, uint64_t out_len, const float* x_host, uint64_t x_len,
                       const goph_mlx_weight* w, int batch);

/* ---- GGUF Q8_0 / Q4_K matrices (loader/gguf/quant_matrix.go, runtime/{q8,q4k,gguf_matrix}.go) */

/* nvidia.UploadGGUFMatrix / UploadQ4KMatrixRaw / UploadQ8_0MatrixRows
 * (runtime/gguf_matrix.go:19-39, q4k.go:172, q8.go:109): raw is the GGUF row-major block
 * stream (34-byte Q8_0 blocks or 144-byte Q4_K super-blocks), out_dim rows of in_dim. */
int goph_gguf_upload(int device, int qtype, const uint8_t* raw, uint64_t raw_len, int in_dim,
                     int out_dim, goph_gguf_matrix** out);
int goph_gguf_free(goph_gguf_matrix* m);
uint64_t goph_gguf_resident_bytes(const goph_gguf_matrix* m);
/* QuantMatrix.DequantRowTo for every row (loader/gguf/quant_matrix.go:42-60), bit-exact. */
int goph_gguf_dequant(const goph_gguf_matrix* m, float* out_dev, uint64_t out_len, void* stream);
/* nvidia.ProjectQ4PairToBuffers (runtime/gguf_matrix.go:82-111): two matrices of one inDim (gate and
 * up) applied to the same x [batch,in]; on the tensor-core path the activations are prepared once
 * for both.  Results equal two goph_gguf_project calls bit for bit. */
int goph_gguf_project_pair(float* out_a_dev, uint64_t out_a_len, float* out_b_dev, uint64_t out_b_len,
                           const float* x_dev, uint64_t x_len, int batch, const goph_gguf_matrix* a,
                           const goph_gguf_matrix* b, void* stream);
/* nvidia.GateUpGELUQ4KBatchToBuffer (runtime/q4k.go:338-352): m holds the gate rows [0, intermediate) and
 * the up rows [intermediate, 2 intermediate); out[b][i] = gelu(gate_i . x_b) * (up_i . x_b) with the tanh
 * form of GELU the reference kernel uses (ptx/q4/gate_up_gelu_q4k.go:157-176).  Q4_K or Q8_0, either layout. */
int goph_gguf_gate_up_gelu(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len, int batch,
                           int intermediate, const goph_gguf_matrix* m, void* stream);
/* nvidia.GateUpGELUQ4KByWorkToBuffer (runtime/q4k.go:322-336): m stacks active_experts slabs of
 * 2 x intermediate rows (gate rows, then up rows); work item w multiplies x[w] by the slab of expert
 * work_experts_dev[w] (u32, device memory).  An index >= active_experts is skipped and sets the kernel
 * status word to 601.  (The pointer-table form, GateUpGELUQ4KByWorkPtrsToBuffer, takes separate
 * matrices; stack them at upload to use this call.)  An expert's rows are read once per
 * four of its items (lists of up to 1024 items, in_dim a multiple of 256; else once per item). */
int goph_gguf_gate_up_gelu_by_work(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                                   const uint32_t* work_experts_dev, int work_len, int intermediate, int active_experts,
                                   const goph_gguf_matrix* m, void* stream);
/* nvidia.GemvQ8_0BatchScatter (runtime/q8.go:209-222): dst[pos[b]][r] += weight[b] * (W[r] . x_b), dst of
 * rows of out_dim floats.  Additions are atomic (rows of dst may be shared between items); a destination
 * past dst_len is skipped and sets the kernel status word to 602. */
int goph_gguf_project_scatter(float* dst_dev, uint64_t dst_len, const float* x_dev, uint64_t x_len,
                              const uint32_t* pos_dev, const float* weight_dev, int batch, const goph_gguf_matrix* m,
                              void* stream);
/* nvidia.GemvQ8_0ScatterByWork (runtime/q8.go:193-207): m stacks active_experts slabs of
 * out_dim / active_experts rows; item w: dst[work_pos[w]][r] += work_weight[w] * (W_e[r] . x_w) with
 * e = work_active[w].  Q8_0 or Q4_K, either layout. */
int goph_gguf_scatter_by_work(float* dst_dev, uint64_t dst_len, const float* x_dev, uint64_t x_len,
                              const uint32_t* work_active_dev, const uint32_t* work_pos_dev,
                              const float* work_weight_dev, int work_len, int active_experts,
                              const goph_gguf_matrix* m, void* stream);
/* GPUGGUFMatrix.ProjectBatchToBuffer / GemvQ4KBatchToBuffer / GemvQ8_0BatchToBuffer
 * (runtime/gguf_matrix.go:121-135, q4k.go:351, q8.go:225): x [batch,in] f32 → out [batch,out]. */
int goph_gguf_project(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                      int batch, const goph_gguf_matrix* m, void* stream);
/* nvidia.GemvQ4K / GemvQ4KBatch / GemvQ8_0 / GemvQ8_0Batch with Go slices
 * (runtime/q4k.go:533-595, q8.go:239-301). */
int goph_gguf_project_host(float* out_host, uint64_t out_len, const float* x_host, uint64_t x_len,
                           int batch, const goph_gguf_matrix* m);

/* ---- product lists: many batch-1 MLX products in one launch -------------------------------
 * The reference launches one kernel per projection (runtime/mlx.go:287-321); at batch 1 the small
 * projections of a decode step are bound by launch latency, not by memory.  A product list is
 * created once from the weights, outputs and activation vectors of consecutive projections and
 * then run as ONE cooperative kernel: every CTA works through the list, with a grid-wide barrier
 * between products, so product k+1 may read (as its x) what product k wrote.  Results are those
 * of goph_mlx_gemv on the same arguments, bit for bit. */
typedef struct goph_mlx_program goph_mlx_program;

/* n_ops products; product o multiplies xs_dev[o] (in_dim f32, 16-byte aligned) with
 * weights_per_op[o] weights (1..8, sharing in_dim and group size; ws and outs_dev are the
 * concatenation over products).  Weights must be in the row-major layout (upload with option
 * "mlx_layout" = 1 or under 8 Mi weights), group size a power of two >= 32, one scale-table
 * format per list.  The buffers are borrowed: they must outlive the list. */
int goph_mlx_program_create(int device, int n_ops, const int* weights_per_op, const goph_mlx_weight* const* ws,
                            float* const* outs_dev, const float* const* xs_dev, goph_mlx_program** out);
/* The same with an operation applied to a product's x while it is staged, as goph_mlx_gemv_pre does for
 * a single launch (arrays of n_ops entries, or NULL for none): pre_ops[o] = 0 none; 1 v = x (+ pre_b[o]),
 * stored to pre_hidden[o] when not NULL, x' = RMSNorm(v) * pre_w[o] with pre_eps[o]; 2 x' = SiLU(x) * pre_b[o].
 * A product's outputs and hidden vector must not overlap what it reads.  With these a decoder layer's
 * o -> (add, norm) gate|up -> (SiLU, mul) down -> (add, norm) next q|k|v is one launch. */
int goph_mlx_program_create_pre(int device, int n_ops, const int* weights_per_op, const goph_mlx_weight* const* ws,
                                float* const* outs_dev, const float* const* xs_dev, const int* pre_ops,
                                const float* const* pre_b, const float* const* pre_w, float* const* pre_hidden,
                                const float* pre_eps, goph_mlx_program** out);
/* Runs the list on `stream` (capturable into a CUDA graph).  Runs of one list must not overlap. */
int goph_mlx_program_run(goph_mlx_program* p, void* stream);
/* 0, or 200 + k when a CTA gave up waiting (about a second) at the barrier in front of product k;
 * the list must then be freed.  Synchronises with the device. */
int goph_mlx_program_status(goph_mlx_program* p, int* out_status);
int goph_mlx_program_free(goph_mlx_program* p);
/* ---- GPTQ symmetric INT4 weights (backends/simd/quant/q4, runtime/q4.go, gemm_q4.go) ---- */

typedef struct goph_gptq_weight goph_gptq_weight; /* nvidia.GPUQuantWeight (runtime/q4.go:18-26) */

/* nvidia.UploadQuantWeight (runtime/q4.go:29-102): qweight [in_dim/8, out_dim] int32 (input 8p+k in
 * bits 4k..4k+3 of row p), g_idx [in_dim], scales [groups, out_dim] with groups = scales_len / out_dim;
 * weight = scale * (q - 8).  Same rejections as the reference: in_dim not a multiple of 8, short
 * buffers, scales_len not a positive multiple of out_dim, g_idx outside [0, groups).
 * A g_idx of equal consecutive groups (group size a multiple of 8) is served by the MLX kernels
 * (q*s - 8*s is that format's affine form), any other g_idx by a row kernel with per-input scale
 * lookup. */
int goph_gptq_upload(int device, const int32_t* qweight, uint64_t qweight_len, const int32_t* g_idx,
                     uint64_t g_idx_len, const float* scales, uint64_t scales_len, int in_dim, int out_dim,
                     goph_gptq_weight** out);
/* GPUQuantWeight.Free (runtime/q4.go:104-120); NULL is a no-op. */
int goph_gptq_free(goph_gptq_weight* w);
uint64_t goph_gptq_resident_bytes(const goph_gptq_weight* w);
/* 1 when the weight is held in the MLX layouts (regular g_idx), 0 otherwise. */
int goph_gptq_uses_mlx_kernels(const goph_gptq_weight* w);
/* nvidia.GemvQ4 (batch 1; runtime/q4.go:149-182) and nvidia.GemmQ4 (runtime/gemm_q4.go:24-68) on device
 * buffers: x [batch,in_dim] f32 -> out [batch,out_dim].  No CPU fallback. */
int goph_gptq_gemm(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len, int batch,
                   const goph_gptq_weight* w, void* stream);
/* q4.DequantSymTo (backends/simd/quant/q4/dequant.go:134-197): [out_dim, in_dim] row-major f32,
 * bit-exact (scale * float32(q - 8)). */
int goph_gptq_dequant(const goph_gptq_weight* w, float* out_dev, uint64_t out_len, void* stream);

/* ---- FP8 E4M3 linears (backends/simd/quant/fp8, runtime/fp8.go) ---------------------- */

/* nvidia.UploadFP8E4M3Linear (runtime/fp8.go:48): weight [out_dim,in_dim] E4M3FN bytes,
 * scale of length 1 (per tensor) or out_dim (per row), bias NULL or [out_dim]. */
int goph_fp8_upload(int device, const uint8_t* weight, uint64_t weight_len, const float* scale,
                    int scale_len, const float* bias, int bias_len, int out_dim, int in_dim,
                    goph_fp8_linear** out);
int goph_fp8_free(goph_fp8_linear* w);
uint64_t goph_fp8_resident_bytes(const goph_fp8_linear* w);
/* fp8.Linear.DequantRowTo for every row (backends/simd/quant/fp8/fp8.go:181-198), bit-exact. */
int goph_fp8_dequant(const goph_fp8_linear* w, float* out_dev, uint64_t out_len, void* stream);
/* nvidia.GemvFP8E4M3Buffer / GemmFP8E4M3Buffer (runtime/fp8.go:995, :271). */
int goph_fp8_gemm(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len, int batch,
                  const goph_fp8_linear* w, void* stream);
/* nvidia.GemmFP8E4M3Buffer (runtime/fp8.go:271-320) for activations held as bf16: x_bf16_dev is
 * [batch,in] bf16 bit patterns, 16-byte aligned; the weights are streamed once per 64 rows.
 * Linears in the tensor-core layout only (GOPH_E_UNSUPPORTED otherwise). */
int goph_fp8_gemm_bf16(float* out_dev, uint64_t out_len, const uint16_t* x_bf16_dev, uint64_t x_len, int batch,
                       const goph_fp8_linear* w, void* stream);
/* nvidia.GemvFP8E4M3 / GemmFP8E4M3 with Go slices (runtime/fp8.go:158, :180). */
int goph_fp8_gemm_host(float* out_host, uint64_t out_len, const float* x_host, uint64_t x_len,
                       int batch, const goph_fp8_linear* w);

/* ---- mixture-of-experts selected-expert projection (MLX 4-bit experts) ------------------ */

/* One MoE layer: its routing constants and device scratch for up to max_tokens tokens per call.
 * Replaces the per-layer state of model.moeForwardGPU (model/moe_gpu.go:49-130): top_k <= 0 means
 * 8 and is clamped to num_experts (model/moe.go:209-215); norm_topk as cfg.NormTopKProb. */
int goph_moe_create(int device, int num_experts, int hidden, int inter, int group_size, int top_k,
                    int norm_topk, int max_tokens, goph_moe_layer** out);
/* Router weight [num_experts x hidden] (LlamaLayer.RouterW uploaded with goph_mlx_upload).  Borrowed. */
int goph_moe_set_router(goph_moe_layer* m, const goph_mlx_weight* router);
/* Expert eid's gate/up [inter x hidden] and down [hidden x inter] weights (borrowed).  The experts
 * of a layer share one device layout: row-major (option "mlx_layout" = 1 at upload, or the default
 * for matrices under 8 Mi weights) runs them on the CUDA cores; tiled ("mlx_layout" = 2 at upload;
 * hidden and inter multiples of 256) runs all selected experts as grouped launches of the
 * tensor-core kernel, which is the faster form from a few tokens per call upwards.
 * All three NULL marks the expert as not resident on this GPU: goph_moe_forward then
 * leaves its contribution out, which is how experts are placed across GPUs
 * (backends/placement/expert_pool.go:101-153 keeps a resident subset; here the subset is per GPU). */
int goph_moe_set_expert(goph_moe_layer* m, int eid, const goph_mlx_weight* gate,
                        const goph_mlx_weight* up, const goph_mlx_weight* down);
int goph_moe_free(goph_moe_layer* m);
/* out[t] = sum over the top-k experts e of token t, in selection order, of
 * weight_e * down_e . (silu(gate_e . x[t]) * (up_e . x[t])) — moeForwardWithREAP
 * (model/moe.go:203-347) / moeForwardGPU (model/moe_gpu.go:49-303) for `tokens` rows of x
 * [tokens x hidden].  Routing runs on the device; nothing is copied to the host. */
int goph_moe_forward(goph_moe_layer* m, float* out_dev, uint64_t out_len, const float* x_dev,
                     uint64_t x_len, int tokens, void* stream);
/* Same with the router logits [tokens x num_experts] supplied by the caller (the selected-expert
 * projection alone: MLXSelectedExpertPersistentCandidate.Run,
 * backends/nvidia/runtime/mlx_selected_expert.go:77-177, fed by routing done elsewhere). */
int goph_moe_forward_logits(goph_moe_layer* m, float* out_dev, uint64_t out_len, const float* x_dev,
                            uint64_t x_len, const float* logits_dev, uint64_t logits_len, int tokens,
                            void* stream);
/* Expert ids (-1 = none) and weights [tokens x top_k] chosen by the last forward call. */
int goph_moe_last_routing(goph_moe_layer* m, int tokens, int* ids_host, float* weights_host);

/* ---- the other operations of a decode step ----------------------------------------------
 * The kernels GPUModel.Generate launches between the projections (model/gpu_forward.go:993-1357),
 * with the arithmetic of runLegacyCPUToken (model/llama.go:899-1441).  The position and the current
 * token are read from device memory, so one captured CUDA graph serves every step. */

/* hidden = a (+ b when b is not NULL; hidden may be NULL); normed = RMSNorm(hidden) * weight, per row
 * of n (simd.RMSNorm, backends/simd/runtime/vec_amd64.s:280-375; the residual add of
 * model/llama.go:1213-1216 in front of it). */
int goph_add_rmsnorm(int device, float* hidden_dev, float* normed_dev, const float* a_dev, const float* b_dev,
                     const float* weight_dev, int n, int rows, float eps, void* stream);
/* Per head: optional QK RMSNorm (Qwen3, model/llama.go:1105-1127), RoPE with the table row of
 * *pos_dev (kernels.ApplyRoPE, backends/simd/kernels/rope.go:29-44; table [max_seq][head_dim/2][cos,sin]
 * as simd.BuildRoPEFreqs makes it); q in place, k and v into row *pos_dev of the caches
 * [max_seq][kv_heads*head_dim] (model/llama.go:1150-1160).  A position outside [0, max_seq) leaves
 * q and the caches untouched and sets the device status word (goph_kernel_status) to 401; the
 * attention entry points below do the same with 402. */
int goph_qk_norm_rope_append(int device, float* q_dev, const float* k_dev, const float* v_dev,
                             const float* q_norm_dev, const float* k_norm_dev, const float* rope_table_dev,
                             const int* pos_dev, float* kcache_dev, float* vcache_dev, int max_seq, int heads,
                             int kv_heads, int head_dim, float eps, void* stream);
/* simd.GQAAttentionScaleInto over positions 0..*pos_dev (backends/simd/runtime/attention.go:82-113). */
int goph_attn_decode(int device, float* out_dev, const float* q_dev, const float* kcache_dev,
                     const float* vcache_dev, const int* pos_dev, int max_seq, int heads, int kv_heads,
                     int head_dim, float scale, void* stream);
/* goph_qk_norm_rope_append and goph_attn_decode in one launch: q_dev, k_dev, v_dev are the raw
 * projection outputs of the current position; the new k and v are also written into their cache rows. */
int goph_attn_decode_fused(int device, float* out_dev, const float* q_dev, const float* k_dev, const float* v_dev,
                           const float* q_norm_dev, const float* k_norm_dev, const float* rope_table_dev,
                           const int* pos_dev, float* kcache_dev, float* vcache_dev, int max_seq, int heads,
                           int kv_heads, int head_dim, float scale, float eps, void* stream);
/* simd.VecSiLUMul (backends/simd/kernels/activation.go:15-24). */
int goph_silu_mul(int device, float* out_dev, const float* gate_dev, const float* up_dev, int n, void* stream);
/* ArgmaxLogits (model/inference_helpers.go:248-261: the first maximum) and the bookkeeping of the
 * greedy loop: *tok_dev = the winner (or forced_dev[*pos_dev + 1] when that is >= 0: prompt tokens),
 * history_dev[*pos_dev + 1] = it, *pos_dev += 1. */
int goph_argmax_advance(int device, const float* logits_dev, int n, int* tok_dev, int* pos_dev, int* history_dev,
                        const int* forced_dev, int history_cap, void* stream);
/* out = W . f(x) with the operation in front of the projection folded into the product's launch:
 *   pre_op 1  v = x (+ b when not NULL); hidden_out = v (optional; must not alias x or b);
 *             f = RMSNorm(v) * norm_w            (residual add + norm + q|k|v or gate|up projection)
 *   pre_op 2  f = silu(x) * b                    (activation + down projection)
 * Row-major MLX weights (group size >= 32), batch 1, 16-byte aligned vectors; otherwise
 * GOPH_E_UNSUPPORTED and the caller issues the operations separately. */
int goph_mlx_gemv_pre(float* out_dev, uint64_t out_len, const goph_mlx_weight* w, int pre_op, const float* x_dev,
                      const float* b_dev, const float* norm_w_dev, float* hidden_out_dev, float eps, void* stream);
/* LlamaModel.TokenEmbeddingInto for a tied MLX LM head: dequantised row *tok_dev (model/inference_helpers.go:20-44). */
int goph_mlx_embed(float* out_dev, uint64_t out_len, const goph_mlx_weight* w, const int* tok_dev, void* stream);

/* ---- row-sharded products across the GPUs of one box ----------------------------------------
 * The reference is single-GPU.  A projection [out x in] is split by rows: rank r of `world` uploads
 * rows [lo, hi) as an ordinary weight handle (rows are contiguous in every format), computes
 * [batch x (hi-lo)], and the blocks are exchanged so that every rank holds [batch x out].  One rank
 * per GPU; ranks may be processes (areas shared through goph_gather_export/open_peer) or live in
 * one process (goph_gather_attach_local).  Every rank must issue the same sequence of exchanges. */

/* Rows [lo, hi) owned by `rank`: contiguous, cut at multiples of `align` rows, the same for every caller. */
int goph_shard_rows(int out_dim, int rank, int world, int align, int* lo, int* hi);
/* Exchange area for results of up to capacity_floats floats (world <= 8). */
int goph_gather_create(int device, int rank, int world, uint64_t capacity_floats, goph_gather** out);
/* 64-byte token by which another process maps this rank's area. */
int goph_gather_export(goph_gather* g, unsigned char* handle64);
int goph_gather_open_peer(goph_gather* g, int peer_rank, const unsigned char* handle64);
/* Same-process form: connects g to the area of `peer` (another rank's handle), enabling peer access. */
int goph_gather_attach_local(goph_gather* g, goph_gather* peer);
int goph_gather_free(goph_gather* g);
/* 0, or 100+q if a block of rank q did not arrive within the wait limit (~2 s).  The waits are
 * bounded; the context stays usable. */
int goph_gather_status(goph_gather* g, int* out_status);
/* Device buffer of capacity_floats floats in which a rank may build its block. */
int goph_gather_shard_buffer(goph_gather* g, float** shard_dev);
/* All ranks' blocks side by side in every rank's result buffer.  A result row is `total` floats
 * wide (row_stride >= total apart); rank q owns columns [q*per, min(total, (q+1)*per)) of it and
 * passes them as src[rows][its width].  *result_dev receives this rank's result buffer
 * [rows x row_stride]; stream-ordered: kernels launched after the call on `stream` see all ranks'
 * blocks, and the buffer is rewritten by the next exchange on this handle. */
int goph_gather_all(goph_gather* g, const float* src_dev, int rows, int per, int64_t total,
                    int64_t row_stride, void* stream, float** result_dev);
/* Sharded product + exchange: `shard` holds the rows goph_shard_rows(out_dim_full, rank, world, 8)
 * gives this rank, starting at row_lo (NULL for a rank that owns no rows); *result_dev receives
 * [batch x out_dim_full] on every rank.
 * (GemmMLX / ProjectBatchToBuffer / GemmFP8E4M3Buffer for a weight split over GPUs.) */
int goph_mlx_gemm_allgather(goph_gather* g, const goph_mlx_weight* shard, const float* x_dev, uint64_t x_len,
                            int batch, int row_lo, int out_dim_full, void* stream, float** result_dev);
int goph_gguf_project_allgather(goph_gather* g, const goph_gguf_matrix* shard, const float* x_dev, uint64_t x_len,
                                int batch, int row_lo, int out_dim_full, void* stream, float** result_dev);
int goph_fp8_gemm_allgather(goph_gather* g, const goph_fp8_linear* shard, const float* x_dev, uint64_t x_len,
                            int batch, int row_lo, int out_dim_full, void* stream, float** result_dev);
/* goph_moe_forward on a layer whose experts are placed per GPU: every rank computes the partial sum
 * of its resident experts, the partials [tokens x hidden] are exchanged and added in rank order. */
int goph_moe_forward_sharded(goph_gather* g, goph_moe_layer* m, float* out_dev, uint64_t out_len,
                             const float* x_dev, uint64_t x_len, int tokens, int hidden, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GOPH_B200_H */
