// All-gather of row-sharded outputs over NVLink peer memory, fused behind the sharded products.
//
// The reference has no multi-GPU path; this is the exchange step that row-sharding a projection
// (or placing MoE experts per GPU) needs: every rank's [M, out/G] block (or partial [T, hidden] sum)
// must reach every other rank.  The blocks are a few KB, so the cost is latency, not bandwidth:
// instead of a library collective the producing rank stores its block straight into every peer's
// result buffer (plain st.global to peer memory mapped through CUDA IPC or peer access), then
// raises a flag in each peer's memory; one thread per GPU waits — bounded — until every peer's
// flag for this exchange has arrived.  One launch per exchange, placed behind the product's
// kernel with programmatic dependent launch.
//
// Memory of one rank's exchange area (one cudaMalloc, exported to the peers):
//   [0, 256)                 uint32 flags[8]: flags[q] = number of the last exchange rank q completed into this area
//   [256, 256 + 4*cap)       result buffer for odd exchanges
//   [256 + 4*cap, ...)       result buffer for even exchanges
// The exchange number lives in device memory (the kernel advances it), so exchanges can be captured
// into a CUDA graph; the result buffer alternates with the number's parity, and since the host hands
// the buffer's address to the readers at capture time, a replayed graph must hold an even number of
// exchanges per exchange area (the kernel flags a mismatch in the status word).
// Two result buffers are enough: a rank can only start exchange e+2 after every peer has raised
// its flag for e+1, which a peer does after (in stream order) its readers of exchange e.
#include <string.h>

#include "goph_internal.cuh"

namespace goph {
constexpr uint32_t kMagicGather = 0x47415448;  // "GATH"
constexpr int kMaxRanks = 8;
constexpr long long kGatherTimeoutCycles = 4000000000ll;  // ~2 s at the maximum SM clock

struct GatherArgs {
  unsigned char* peer[kMaxRanks];
  int world, rank;
  int expected_parity;      // parity of the exchange number the host believes this launch has
  unsigned long long cap_bytes;
  const float* src;
  int rows, count;
  long long dst_off, dst_row_stride;
  int* done;                // arrival counter
  int* status;
  uint32_t* epoch_dev;      // number of exchanges completed on this rank; the kernel numbers itself from it
};

__global__ void __launch_bounds__(256) gather_push_kernel(GatherArgs a) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // The exchange numbers itself on the device, so a captured graph can be replayed.  Every CTA reads
  // the counter before the last one to arrive advances it.
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_dev) + 1;
  const unsigned long long buf_off = 256 + (unsigned long long)(epoch & 1) * a.cap_bytes;
  const long long total = (long long)a.rows * a.count;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  const bool vec = a.count % 4 == 0 && a.dst_off % 4 == 0 && a.dst_row_stride % 4 == 0 && ((uintptr_t)a.src & 15) == 0;
  for (int p = 0; p < a.world; ++p) {
    const int q = (a.rank + p) % a.world;  // start with the own copy, then walk the peers in a rank-dependent order
    float* dst = reinterpret_cast<float*>(a.peer[q] + buf_off) + a.dst_off;
    if (vec) {
      const int c4 = a.count / 4;
      for (long long i = tid; i < total / 4; i += nth) {
        const long long m = i / c4, j = i - m * c4;
        float4 v = reinterpret_cast<const float4*>(a.src)[i];
        *reinterpret_cast<float4*>(dst + m * a.dst_row_stride + j * 4) = v;
      }
    } else {
      for (long long i = tid; i < total; i += nth) {
        const long long m = i / a.count, j = i - m * a.count;
        dst[m * a.dst_row_stride + j] = a.src[i];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(a.done, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!s_last || threadIdx.x >= 32) return;
  // last CTA, first warp: lane q signals rank q and waits for rank q's signal
  __threadfence_system();
  if (threadIdx.x == 0) {
    *a.done = 0;
    *a.epoch_dev = epoch;
    // the host handed out the result buffer of the other parity: its count of exchanges is off
    // (a replayed graph must hold an even number of exchanges)
    if ((int)(epoch & 1) != a.expected_parity) atomicCAS(a.status, 0, 200);
  }
  const int q = threadIdx.x;
  if (q < a.world) {
    uint32_t* remote = reinterpret_cast<uint32_t*>(a.peer[q]) + a.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const uint32_t* local = reinterpret_cast<const uint32_t*>(a.peer[a.rank]) + q;
    const long long t0 = clock64();
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local) : "memory");
      if ((int)(v - epoch) >= 0) break;
      if (clock64() - t0 > kGatherTimeoutCycles) {
        atomicCAS(a.status, 0, 100 + q);  // rank q's block never arrived
        break;
      }
      __nanosleep(100);
    }
  }
}

// out[i] = sum over ranks r = 0..world-1, in that order, of gathered[r*count + i]
__global__ void gather_sum_kernel(const float* __restrict__ gathered, float* __restrict__ out, long long count, int world) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) acc = __fadd_rn(acc, gathered[(size_t)r * count + i]);
    out[i] = acc;
  }
}
}  // namespace goph

struct goph_gather {
  uint32_t magic;
  int device, rank, world;
  uint64_t capacity;  // floats per result buffer
  unsigned char* area;
  unsigned char* peer[goph::kMaxRanks];
  int peer_kind[goph::kMaxRanks];  // 0 not connected, 1 opened from an IPC handle, 2 this process's memory
  uint32_t epoch;
  int* done;    // [0] arrival counter, [1] status, [2] exchanges completed
  float* shard; // this rank's block before it is pushed [capacity]
};

using namespace goph;

static bool valid_gather(const goph_gather* g) { return g && g->magic == kMagicGather; }

GOPH_API int goph_shard_rows(int out_dim, int rank, int world, int align, int* lo, int* hi) {
  clear_error();
  if (out_dim < 0 || world <= 0 || rank < 0 || rank >= world || align <= 0 || !lo || !hi)
    return fail(GOPH_E_INVALID, "goph_shard_rows: out_dim=%d rank=%d world=%d align=%d", out_dim, rank, world, align);
  long long blocks = ((long long)out_dim + align - 1) / align;
  long long per = (blocks + world - 1) / world * align;
  long long l = (long long)rank * per, h = l + per;
  if (l > out_dim) l = out_dim;
  if (h > out_dim) h = out_dim;
  *lo = (int)l;
  *hi = (int)h;
  return GOPH_OK;
}

GOPH_API int goph_gather_create(int device, int rank, int world, uint64_t capacity_floats, goph_gather** out) {
  clear_error();
  if (!out) return fail(GOPH_E_INVALID, "goph_gather_create: nil result pointer");
  *out = nullptr;
  if (world <= 0 || world > kMaxRanks || rank < 0 || rank >= world || capacity_floats == 0 || capacity_floats > (1ull << 32))
    return fail(GOPH_E_INVALID, "goph_gather_create: rank=%d world=%d (max %d) capacity=%llu", rank, world, kMaxRanks,
                (unsigned long long)capacity_floats);
  if (int rc = use_device(device)) return rc;
  capacity_floats = (capacity_floats + 63) / 64 * 64;
  goph_gather* g = new goph_gather();
  memset(g, 0, sizeof *g);
  g->device = device;
  g->rank = rank;
  g->world = world;
  g->capacity = capacity_floats;
  const size_t bytes = 256 + 2 * capacity_floats * sizeof(float);
  cudaError_t e = cudaMalloc(&g->area, bytes);
  if (e == cudaSuccess) e = cudaMemset(g->area, 0, bytes);
  if (e == cudaSuccess) e = cudaMalloc(&g->done, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(g->done, 0, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(&g->shard, capacity_floats * sizeof(float));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // the area is zero before any peer can see it
  if (e != cudaSuccess) {
    cudaFree(g->area);
    cudaFree(g->done);
    cudaFree(g->shard);
    delete g;
    return fail_cuda(e, "cudaMalloc(exchange area)");
  }
  g->peer[rank] = g->area;
  g->peer_kind[rank] = 2;
  g->magic = kMagicGather;
  *out = g;
  return GOPH_OK;
}

GOPH_API int goph_gather_export(goph_gather* g, unsigned char* handle64) {
  clear_error();
  if (!valid_gather(g) || !handle64) return fail(GOPH_E_INVALID, "goph_gather_export: invalid handle");
  if (int rc = use_device(g->device)) return rc;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  GOPH_CUDA(cudaIpcGetMemHandle(&h, g->area));
  memcpy(handle64, &h, 64);
  return GOPH_OK;
}

GOPH_API int goph_gather_open_peer(goph_gather* g, int peer_rank, const unsigned char* handle64) {
  clear_error();
  if (!valid_gather(g) || !handle64) return fail(GOPH_E_INVALID, "goph_gather_open_peer: invalid handle");
  if (peer_rank < 0 || peer_rank >= g->world || peer_rank == g->rank || g->peer_kind[peer_rank])
    return fail(GOPH_E_INVALID, "goph_gather_open_peer: rank %d is out of range, this rank, or already connected", peer_rank);
  if (int rc = use_device(g->device)) return rc;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  GOPH_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  g->peer[peer_rank] = static_cast<unsigned char*>(p);
  g->peer_kind[peer_rank] = 1;
  return GOPH_OK;
}

GOPH_API int goph_gather_attach_local(goph_gather* g, goph_gather* peer) {
  clear_error();
  if (!valid_gather(g) || !valid_gather(peer)) return fail(GOPH_E_INVALID, "goph_gather_attach_local: invalid handle");
  if (peer->world != g->world || peer->capacity != g->capacity || peer->rank == g->rank || g->peer_kind[peer->rank])
    return fail(GOPH_E_INVALID, "goph_gather_attach_local: peer does not belong to this exchange or is already connected");
  if (int rc = use_device(g->device)) return rc;
  if (peer->device != g->device) {
    int can = 0;
    GOPH_CUDA(cudaDeviceCanAccessPeer(&can, g->device, peer->device));
    if (!can) return fail(GOPH_E_UNSUPPORTED, "device %d cannot address device %d's memory", g->device, peer->device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer->device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      cudaGetLastError();
    } else if (e != cudaSuccess) {
      return fail_cuda(e, "cudaDeviceEnablePeerAccess");
    }
  }
  g->peer[peer->rank] = peer->area;
  g->peer_kind[peer->rank] = 2;
  return GOPH_OK;
}

GOPH_API int goph_gather_free(goph_gather* g) {
  clear_error();
  if (!g) return GOPH_OK;
  if (!valid_gather(g)) return fail(GOPH_E_INVALID, "goph_gather_free: not an exchange handle");
  if (int rc = use_device(g->device)) return rc;
  cudaDeviceSynchronize();
  for (int r = 0; r < g->world; ++r)
    if (g->peer_kind[r] == 1) cudaIpcCloseMemHandle(g->peer[r]);
  cudaFree(g->area);
  cudaFree(g->done);
  cudaFree(g->shard);
  g->magic = 0;
  delete g;
  return GOPH_OK;
}

GOPH_API int goph_gather_status(goph_gather* g, int* out_status) {
  clear_error();
  if (!valid_gather(g) || !out_status) return fail(GOPH_E_INVALID, "goph_gather_status: invalid handle");
  if (int rc = use_device(g->device)) return rc;
  GOPH_CUDA(cudaMemcpy(out_status, g->done + 1, sizeof(int), cudaMemcpyDeviceToHost));
  return GOPH_OK;
}

GOPH_API int goph_gather_shard_buffer(goph_gather* g, float** shard_dev) {
  clear_error();
  if (!valid_gather(g) || !shard_dev) return fail(GOPH_E_INVALID, "goph_gather_shard_buffer: invalid handle");
  *shard_dev = g->shard;
  return GOPH_OK;
}

GOPH_API int goph_gather_all(goph_gather* g, const float* src_dev, int rows, int count, int64_t dst_off,
                             int64_t dst_row_stride, void* stream, float** result_dev) {
  clear_error();
  if (!valid_gather(g)) return fail(GOPH_E_INVALID, "goph_gather_all: invalid handle");
  if ((!src_dev && count > 0) || rows <= 0 || count < 0 || dst_off < 0 || dst_row_stride < count || !result_dev)
    return fail(GOPH_E_INVALID, "goph_gather_all: rows=%d count=%d offset=%lld stride=%lld", rows, count, (long long)dst_off,
                (long long)dst_row_stride);
  if ((uint64_t)dst_off + (uint64_t)(rows - 1) * (uint64_t)dst_row_stride + (uint64_t)count > g->capacity)
    return fail(GOPH_E_INVALID, "goph_gather_all: block ends past the exchange capacity of %llu floats", (unsigned long long)g->capacity);
  for (int r = 0; r < g->world; ++r)
    if (!g->peer_kind[r]) return fail(GOPH_E_INVALID, "goph_gather_all: rank %d is not connected", r);
  if (int rc = use_device(g->device)) return rc;
  GatherArgs a;
  memset(&a, 0, sizeof a);
  for (int r = 0; r < g->world; ++r) a.peer[r] = g->peer[r];
  a.world = g->world;
  a.rank = g->rank;
  const uint32_t epoch = ++g->epoch;  // host mirror; the device counter is the one the kernels use
  a.expected_parity = (int)(epoch & 1);
  a.cap_bytes = g->capacity * sizeof(float);
  a.epoch_dev = reinterpret_cast<uint32_t*>(g->done + 2);
  a.src = src_dev;
  a.rows = rows;
  a.count = count;
  a.dst_off = dst_off;
  a.dst_row_stride = dst_row_stride;
  a.done = g->done;
  a.status = g->done + 1;
  long long total = (long long)rows * count;
  int grid = (int)((total / 4 + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > 32) grid = 32;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, gather_push_kernel, a));
  *result_dev = reinterpret_cast<float*>(g->area + 256 + (uint64_t)(epoch & 1) * a.cap_bytes);
  return GOPH_OK;
}

static int check_shard(const goph_gather* g, int shard_out, int batch, int row_lo, int out_dim_full) {
  if (!valid_gather(g)) return fail(GOPH_E_INVALID, "invalid exchange handle");
  if (batch <= 0 || row_lo < 0 || shard_out < 0 || (int64_t)row_lo + shard_out > out_dim_full)
    return fail(GOPH_E_INVALID, "shard rows [%d,%d) do not lie in 0..%d", row_lo, row_lo + shard_out, out_dim_full);
  if ((uint64_t)batch * (uint64_t)out_dim_full > g->capacity)
    return fail(GOPH_E_INVALID, "result [%d x %d] exceeds the exchange capacity of %llu floats", batch, out_dim_full,
                (unsigned long long)g->capacity);
  return GOPH_OK;
}

GOPH_API int goph_mlx_gemm_allgather(goph_gather* g, const goph_mlx_weight* shard, const float* x_dev, uint64_t x_len,
                                     int batch, int row_lo, int out_dim_full, void* stream, float** result_dev) {
  clear_error();
  if (!shard) return fail(GOPH_E_INVALID, "nil weight shard");
  if (int rc = check_shard(g, shard->out_dim, batch, row_lo, out_dim_full)) return rc;
  if (int rc = goph_mlx_gemm(g->shard, (uint64_t)batch * shard->out_dim, x_dev, x_len, shard, batch, stream)) return rc;
  return goph_gather_all(g, g->shard, batch, shard->out_dim, row_lo, out_dim_full, stream, result_dev);
}

GOPH_API int goph_gguf_project_allgather(goph_gather* g, const goph_gguf_matrix* shard, const float* x_dev, uint64_t x_len,
                                         int batch, int row_lo, int out_dim_full, void* stream, float** result_dev) {
  clear_error();
  if (!shard) return fail(GOPH_E_INVALID, "nil matrix shard");
  if (int rc = check_shard(g, shard->out_dim, batch, row_lo, out_dim_full)) return rc;
  if (int rc = goph_gguf_project(g->shard, (uint64_t)batch * shard->out_dim, x_dev, x_len, batch, shard, stream)) return rc;
  return goph_gather_all(g, g->shard, batch, shard->out_dim, row_lo, out_dim_full, stream, result_dev);
}

GOPH_API int goph_fp8_gemm_allgather(goph_gather* g, const goph_fp8_linear* shard, const float* x_dev, uint64_t x_len,
                                     int batch, int row_lo, int out_dim_full, void* stream, float** result_dev) {
  clear_error();
  if (!shard) return fail(GOPH_E_INVALID, "nil linear shard");
  if (int rc = check_shard(g, shard->out_dim, batch, row_lo, out_dim_full)) return rc;
  if (int rc = goph_fp8_gemm(g->shard, (uint64_t)batch * shard->out_dim, x_dev, x_len, batch, shard, stream)) return rc;
  return goph_gather_all(g, g->shard, batch, shard->out_dim, row_lo, out_dim_full, stream, result_dev);
}

GOPH_API int goph_moe_forward_sharded(goph_gather* g, goph_moe_layer* m, float* out_dev, uint64_t out_len,
                                      const float* x_dev, uint64_t x_len, int tokens, int hidden, void* stream) {
  clear_error();
  if (!valid_gather(g)) return fail(GOPH_E_INVALID, "invalid exchange handle");
  if (tokens <= 0 || hidden <= 0) return fail(GOPH_E_INVALID, "tokens=%d hidden=%d", tokens, hidden);
  const uint64_t n = (uint64_t)tokens * hidden;
  if (n * g->world > g->capacity) return fail(GOPH_E_INVALID, "partial sums [%d x %d x %d] exceed the exchange capacity", g->world, tokens, hidden);
  if (!out_dev || out_len < n) return fail(GOPH_E_INVALID, "MoE out length=%llu, want %llu", (unsigned long long)out_len, (unsigned long long)n);
  if (int rc = goph_moe_forward(m, g->shard, n, x_dev, x_len, tokens, stream)) return rc;
  float* gathered = nullptr;
  if (int rc = goph_gather_all(g, g->shard, 1, (int)n, (int64_t)g->rank * n, (int64_t)n * g->world, stream, &gathered)) return rc;
  int grid = (int)((n + 255) / 256);
  if (grid > 592) grid = 592;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, gather_sum_kernel, (const float*)gathered, out_dev, (long long)n, g->world));
  return GOPH_OK;
}
