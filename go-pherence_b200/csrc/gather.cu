// All-gather of row-sharded outputs over NVLink peer memory, fused behind the sharded products.
//
// The reference has no multi-GPU path; this is the exchange step that row-sharding a projection
// (or placing MoE experts per GPU) needs: every rank's [M, out/G] block (or partial [T, hidden] sum)
// must reach every other rank.  The blocks are a few KB, so the cost is latency, not bandwidth.
// Instead of a library collective, one kernel per exchange:
//   push  every value of this rank's block is stored, paired with the exchange number, as one
//         8-byte word {value, number} straight into every peer's receive area (plain st.global to
//         peer memory mapped through CUDA IPC or peer access).  An 8-byte store arrives whole, so
//         the number doubles as the "this word is valid" flag: no fence, no separate signal, no
//         acknowledgement round trip.
//   pull  the same kernel then reads its own receive area: each thread spins — bounded — on the
//         words it is responsible for until they carry this exchange's number, and writes the
//         values into the rank's plain result buffer.  The own block is copied directly.
// The kernel sits behind the product's kernel with programmatic dependent launch; kernels launched
// after it on the stream see the complete result.
//
// Receive area of one rank (one cudaMalloc, exported to the peers): two banks of `cap` 8-byte words;
// exchange number e uses bank e & 1.  Two banks are enough: a peer can run at most one exchange
// ahead of this rank (it cannot finish exchange e+1 without this rank's e+1 block), so while this
// rank reads bank e & 1 a peer writes bank (e+1) & 1 at the latest.  Words are never cleared: a
// 32-bit exchange number does not come round again within any realistic run.  The number lives in
// device memory and is advanced by the kernel itself, so a captured CUDA graph can be replayed.
// The result buffer is private to the rank and single: stream order already separates its readers
// from the next exchange's writes.
#include <string.h>

#include "goph_internal.cuh"

namespace goph {
constexpr uint32_t kMagicGather = 0x47415448;  // "GATH"
constexpr int kMaxRanks = 8;
constexpr long long kGatherTimeoutCycles = 4000000000ll;  // ~2 s at the maximum SM clock

struct GatherArgs {
  unsigned long long* peer[kMaxRanks];  // receive areas (peer[rank] is this rank's own)
  int world, rank;
  unsigned long long cap;   // words per bank
  const float* src;         // this rank's block [rows][my_count]
  float* result;            // [rows][row_stride]
  int rows;
  int per;                  // block width of every rank but possibly the last ones
  long long total;          // valid width of a result row: rank q holds [q*per, min(total, (q+1)*per))
  long long row_stride;
  int* done;                // arrival counter
  int* status;
  uint32_t* epoch_dev;      // number of exchanges completed on this rank
};

__device__ __forceinline__ int block_count(const GatherArgs& a, int q) {
  long long lo = (long long)q * a.per, hi = lo + a.per;
  if (hi > a.total) hi = a.total;
  return hi > lo ? (int)(hi - lo) : 0;
}

__global__ void __launch_bounds__(256) gather_exchange_kernel(const __grid_constant__ GatherArgs a) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // Every CTA reads the counter before the last one to finish advances it.
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_dev) + 1;
  const unsigned long long bank = (unsigned long long)(epoch & 1) * a.cap;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  // ---- push: own block to the own result and, tagged, to every peer's bank ----------------
  const int my_count = block_count(a, a.rank);
  const long long my_off = (long long)a.rank * a.per;
  for (long long i = tid; i < (long long)a.rows * my_count; i += nth) {
    const long long m = i / my_count, j = i - m * my_count;
    const float v = a.src[i];
    const long long at = m * a.row_stride + my_off + j;
    a.result[at] = v;
    const unsigned long long word = ((unsigned long long)epoch << 32) | __float_as_uint(v);
    for (int p = 1; p < a.world; ++p) {
      const int q = (a.rank + p) % a.world;  // each rank walks the peers in its own order
      a.peer[q][bank + at] = word;
    }
  }
  // ---- pull: the peers' blocks out of the own bank ------------------------------------------
  const unsigned long long* mine = a.peer[a.rank] + bank;
  const long long t0 = clock64();
  bool gave_up = false;
  for (int p = 1; p < a.world && !gave_up; ++p) {
    const int q = (a.rank + p) % a.world;
    const int cnt = block_count(a, q);
    const long long off = (long long)q * a.per;
    for (long long i = tid; i < (long long)a.rows * cnt; i += nth) {
      const long long m = i / cnt, j = i - m * cnt;
      const long long at = m * a.row_stride + off + j;
      unsigned long long word;
      while (true) {
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(mine + at) : "memory");
        if ((uint32_t)(word >> 32) == epoch) break;
        if (clock64() - t0 > kGatherTimeoutCycles) {
          atomicCAS(a.status, 0, 100 + q);  // rank q's block did not arrive
          gave_up = true;
          break;
        }
      }
      if (gave_up) break;
      a.result[at] = __uint_as_float((uint32_t)word);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(a.done, 1) == (int)gridDim.x - 1) {
    *a.done = 0;
    *a.epoch_dev = epoch;
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
  uint64_t capacity;            // floats in a result, words per bank
  unsigned long long* area;     // receive area: two banks
  unsigned long long* peer[goph::kMaxRanks];
  int peer_kind[goph::kMaxRanks];  // 0 not connected, 1 opened from an IPC handle, 2 this process's memory
  int* done;      // [0] arrival counter, [1] status, [2] exchanges completed
  float* result;  // [capacity]
  float* shard;   // this rank's block before it is pushed [capacity]
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
  if (world <= 0 || world > kMaxRanks || rank < 0 || rank >= world || capacity_floats == 0 || capacity_floats > (1ull << 30))
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
  const size_t bytes = 2 * capacity_floats * sizeof(unsigned long long);
  cudaError_t e = cudaMalloc(&g->area, bytes);
  if (e == cudaSuccess) e = cudaMemset(g->area, 0, bytes);  // number 0 is never used by an exchange
  if (e == cudaSuccess) e = cudaMalloc(&g->done, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(g->done, 0, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(&g->result, capacity_floats * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&g->shard, capacity_floats * sizeof(float));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // the area is zero before any peer can see it
  if (e != cudaSuccess) {
    cudaFree(g->area);
    cudaFree(g->done);
    cudaFree(g->result);
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
  g->peer[peer_rank] = static_cast<unsigned long long*>(p);
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
  cudaFree(g->result);
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

GOPH_API int goph_gather_all(goph_gather* g, const float* src_dev, int rows, int per, int64_t total,
                             int64_t row_stride, void* stream, float** result_dev) {
  clear_error();
  if (!valid_gather(g)) return fail(GOPH_E_INVALID, "goph_gather_all: invalid handle");
  if (rows <= 0 || per <= 0 || total < 0 || row_stride < total || total > (int64_t)per * g->world || !result_dev)
    return fail(GOPH_E_INVALID, "goph_gather_all: rows=%d per=%d total=%lld stride=%lld world=%d", rows, per, (long long)total,
                (long long)row_stride, g->world);
  if ((uint64_t)rows * (uint64_t)row_stride > g->capacity)
    return fail(GOPH_E_INVALID, "goph_gather_all: result [%d x %lld] exceeds the exchange capacity of %llu floats", rows,
                (long long)row_stride, (unsigned long long)g->capacity);
  const int64_t my_lo = (int64_t)g->rank * per;
  const int64_t my_count = my_lo >= total ? 0 : (total - my_lo < per ? total - my_lo : per);
  if (!src_dev && my_count > 0) return fail(GOPH_E_INVALID, "goph_gather_all: nil block");
  for (int r = 0; r < g->world; ++r)
    if (!g->peer_kind[r]) return fail(GOPH_E_INVALID, "goph_gather_all: rank %d is not connected", r);
  if (int rc = use_device(g->device)) return rc;
  GatherArgs a;
  memset(&a, 0, sizeof a);
  for (int r = 0; r < g->world; ++r) a.peer[r] = g->peer[r];
  a.world = g->world;
  a.rank = g->rank;
  a.cap = g->capacity;
  a.src = src_dev;
  a.result = g->result;
  a.rows = rows;
  a.per = per;
  a.total = total;
  a.row_stride = row_stride;
  a.done = g->done;
  a.status = g->done + 1;
  a.epoch_dev = reinterpret_cast<uint32_t*>(g->done + 2);
  // enough threads that nobody polls more than a few words in sequence
  long long elems = (long long)rows * total;
  int grid = (int)((elems + 256 * 4 - 1) / (256 * 4));
  if (grid < 1) grid = 1;
  const int cap_grid = 2 * device_state(g->device).sm_count;
  if (grid > cap_grid) grid = cap_grid;
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
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, gather_exchange_kernel, a));
  *result_dev = g->result;
  return GOPH_OK;
}

// The partition goph_shard_rows gives: block width and this rank's rows.
static int check_shard(const goph_gather* g, int shard_out, int batch, int row_lo, int out_dim_full, int* per) {
  if (!valid_gather(g)) return fail(GOPH_E_INVALID, "invalid exchange handle");
  if (batch <= 0 || out_dim_full <= 0) return fail(GOPH_E_INVALID, "batch=%d out_dim=%d", batch, out_dim_full);
  int lo = 0, hi = 0, lo0 = 0, hi0 = 0;
  if (int rc = goph_shard_rows(out_dim_full, g->rank, g->world, 8, &lo, &hi)) return rc;
  if (int rc = goph_shard_rows(out_dim_full, 0, g->world, 8, &lo0, &hi0)) return rc;
  if (row_lo != lo || shard_out != hi - lo)
    return fail(GOPH_E_INVALID, "shard holds rows [%d,%d); rank %d of %d owns [%d,%d) of %d (goph_shard_rows, align 8)", row_lo,
                row_lo + shard_out, g->rank, g->world, lo, hi, out_dim_full);
  if ((uint64_t)batch * (uint64_t)out_dim_full > g->capacity)
    return fail(GOPH_E_INVALID, "result [%d x %d] exceeds the exchange capacity of %llu floats", batch, out_dim_full,
                (unsigned long long)g->capacity);
  *per = hi0 - lo0;
  return GOPH_OK;
}

GOPH_API int goph_mlx_gemm_allgather(goph_gather* g, const goph_mlx_weight* shard, const float* x_dev, uint64_t x_len,
                                     int batch, int row_lo, int out_dim_full, void* stream, float** result_dev) {
  clear_error();
  int per = 0;
  if (int rc = check_shard(g, shard ? shard->out_dim : 0, batch, row_lo, out_dim_full, &per)) return rc;
  if (shard)
    if (int rc = goph_mlx_gemm(g->shard, (uint64_t)batch * shard->out_dim, x_dev, x_len, shard, batch, stream)) return rc;
  return goph_gather_all(g, g->shard, batch, per, out_dim_full, out_dim_full, stream, result_dev);
}

GOPH_API int goph_gguf_project_allgather(goph_gather* g, const goph_gguf_matrix* shard, const float* x_dev, uint64_t x_len,
                                         int batch, int row_lo, int out_dim_full, void* stream, float** result_dev) {
  clear_error();
  int per = 0;
  if (int rc = check_shard(g, shard ? shard->out_dim : 0, batch, row_lo, out_dim_full, &per)) return rc;
  if (shard)
    if (int rc = goph_gguf_project(g->shard, (uint64_t)batch * shard->out_dim, x_dev, x_len, batch, shard, stream)) return rc;
  return goph_gather_all(g, g->shard, batch, per, out_dim_full, out_dim_full, stream, result_dev);
}

GOPH_API int goph_fp8_gemm_allgather(goph_gather* g, const goph_fp8_linear* shard, const float* x_dev, uint64_t x_len,
                                     int batch, int row_lo, int out_dim_full, void* stream, float** result_dev) {
  clear_error();
  int per = 0;
  if (int rc = check_shard(g, shard ? shard->out_dim : 0, batch, row_lo, out_dim_full, &per)) return rc;
  if (shard)
    if (int rc = goph_fp8_gemm(g->shard, (uint64_t)batch * shard->out_dim, x_dev, x_len, batch, shard, stream)) return rc;
  return goph_gather_all(g, g->shard, batch, per, out_dim_full, out_dim_full, stream, result_dev);
}

GOPH_API int goph_moe_forward_sharded(goph_gather* g, goph_moe_layer* m, float* out_dev, uint64_t out_len,
                                      const float* x_dev, uint64_t x_len, int tokens, int hidden, void* stream) {
  clear_error();
  if (!valid_gather(g)) return fail(GOPH_E_INVALID, "invalid exchange handle");
  if (tokens <= 0 || hidden <= 0) return fail(GOPH_E_INVALID, "tokens=%d hidden=%d", tokens, hidden);
  const uint64_t n = (uint64_t)tokens * hidden;
  if (n * g->world > g->capacity || n > 0x7fffffffull)
    return fail(GOPH_E_INVALID, "partial sums [%d x %d x %d] exceed the exchange capacity", g->world, tokens, hidden);
  if (!out_dev || out_len < n) return fail(GOPH_E_INVALID, "MoE out length=%llu, want %llu", (unsigned long long)out_len, (unsigned long long)n);
  if (int rc = goph_moe_forward(m, g->shard, n, x_dev, x_len, tokens, stream)) return rc;
  float* gathered = nullptr;
  if (int rc = goph_gather_all(g, g->shard, 1, (int)n, (int64_t)n * g->world, (int64_t)n * g->world, stream, &gathered)) return rc;
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
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, gather_sum_kernel, (const float*)gathered, out_dev, (long long)n, g->world));
  return GOPH_OK;
}
