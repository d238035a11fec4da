// Small-batch products on the 5th-generation tensor cores: bf16 operands, f32 accumulators in TMEM,
// the weights streamed ONCE per pass of up to 64 activation rows.
//
// Stands behind nvidia.GemmMLX (backends/nvidia/runtime/mlx.go:395-431; kernel text
// backends/nvidia/ptx/mlx/mlx.go:179-308, which re-reads the weights for every batch row) and
// nvidia.GemmFP8E4M3Buffer (backends/nvidia/runtime/fp8.go:271-320; ptx/fp8/fp8.go:154-309) for
// prefill chunks and verifier batches.
//
// Arithmetic
//   * A operand (weights, M = 128 rows of a tile): written to TMEM as bf16 by converter warps.
//       MLX 4-bit: nibble n becomes the bf16 16 + n (bits 0x4180 | n << 3: two shifts-and-masks per
//       pair of nibbles, exact).  The 16 is taken out again through the group's sum of x.
//       FP8 E4M3:  the byte's exponent and mantissa are placed into a bf16 and multiplied by 2^120
//       (one packed bf16 multiply per two weights) — exact for normals and subnormals alike.
//   * B operand (activations, N = 16/32/64 columns): bf16.  Activations that are bf16 values go in
//       as they are (one piece); general f32 activations are split into three bf16 pieces
//       hi + mid + lo = x exactly, and the three products accumulate into the same columns.
//   * Every product n * x_piece is exact in f32; the tensor core accumulates in f32.
//   * MLX: one accumulator block per 64-element group (four K = 16 instructions accumulate);
//       the epilogue forms scale * (D - 16 * sum x) + bias * sum x = scale * D + (bias - 16 scale) * sum x
//       per (row, group) in f32 and keeps running sums in registers — mlx.GemvTo's expression
//       (backends/mlx/gemv.go:178-209) with the dot product taken by the tensor core.
//     FP8: one accumulator block per 256-element stage; the epilogue adds the stages in f32 and
//       applies the row scale and bias once at the end (fp8.Linear.GemvTo,
//       backends/simd/quant/fp8/fp8.go:219-239).
//
// Pipeline of one CTA (26 warps, one persistent CTA per SM, walking (128-row tile, K split,
// 256-element chunk) stages; a stage is handed from role to role in two units of half its K steps,
// so the MMAs of the first unit run while the second is still being converted):
//   producer warp    one bulk copy of the weight block (the tiled layouts store a stage's
//                    shared-memory image contiguously), one of the chunk's B tile(s), one of the
//                    chunk's sums of x (MLX), into a ring guarded by full/empty mbarriers; weight
//                    copies are issued before the kernel in front has finished, the first two
//                    stages at once and the rest of the ring when the first has landed.  The
//                    chunk order rotates from tile to tile, so CTAs that run side by side do not
//                    all ask for the same activation tile at the same moment.
//   8 converter warps  all on every stage, thread = (row, K half): swizzled LDS.128 -> bf16 pairs
//                    -> tcgen05.st into one of two 128-column A buffers.
//   MMA warp         waits as a warp, one elected lane issues the stage's tcgen05.mma kind::f16
//                    (M128 x N x K16, A from TMEM, B through a shared-memory descriptor) unit by
//                    unit; tcgen05.commit releases the A buffer, the stage and (per group block /
//                    per item) the accumulators to the epilogue.
//   16 epilogue warps four per TMEM lane quarter, each owning a quarter of the columns:
//                    tcgen05.ld, scales from the staged block, running sums in registers.  K
//                    splits write partial sums to scratch; the CTA arriving last adds them in
//                    split order.
// mbarrier arrivals are one per warp.  Every wait is bounded (~2 s); a waiter that gives up
// records a code (300+) in the status word and the CTA winds down.
#include <string.h>

#include <mutex>

#include "goph_internal.cuh"
#include "tc_common.cuh"
#include "tc_gemm.cuh"

namespace goph {

using namespace tc;

namespace {

// Tuning build only (-DGOPH_TUNING): CTA 0 adds up, per role, the cycles spent in each barrier wait
// and in each phase of its loop; goph_tuning_probe copies the counters out.  The shipped library
// is built without it.
#ifdef GOPH_TUNING
__device__ unsigned long long g_tc_span[4];  // globaltimer ns: min CTA entry, max CTA set-up done, max CTA exit, min set-up done
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ long long g_tc_trace[8][64];  // [event][stage] clock64 of one CTA in the middle of the grid
#define TP(...) __VA_ARGS__
#define DBG(bit) (a.dbg & (bit))
#else
#define TP(...)
#define DBG(bit) 0
#endif

constexpr int kTileRows = 128;
constexpr int kChunkK = 256;
enum { G_MLX4 = 0, G_FP8 = 1 };

constexpr int kConvWarps = 8, kEpiWarps = 16;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kWarpTMA = kConvWarps + kEpiWarps, kWarpMMA = kWarpTMA + 1;
constexpr int kMmaWarps = 1;
constexpr int kThreads = (kWarpMMA + kMmaWarps) * 32;
constexpr int kMlxWBytes = kTileRows * 128 + kTileRows * 16;  // nibbles + {scale,bias} pairs of a stage
constexpr int kFp8WBytes = kTileRows * 256;

struct GemmArgs {
  const unsigned char* w;    // tiled weight blocks [tile][chunk]
  const unsigned char* xb;   // B tiles [chunk][piece][K step 16][K half 2][NC/8][8 rows][16 B]
  const float* xtab;         // MLX: [chunk][4 groups][NC] sums of x
  const float* scale;        // FP8: [out_dim]
  const float* bias;         // FP8: [out_dim] or nullptr
  float* out;                // [batch][out_dim]
  int* status;
  float* scratch;            // split-K partial sums [tile][split][NC][128]
  unsigned int* counters;    // per-tile arrival counters, zero between launches
  int out_dim, in_dim, batch;
  int ntiles, nchunks, splits, items, stages;
  int cluster;               // 1: the K splits of a tile are the CTAs of a thread-block cluster (one item each); partial sums through the first CTA's shared memory
  int rotate;                // 1: every tile starts its K range at a different chunk (see StageWalk::chunk)
  int dbg;                   // tuning build only: parts of the kernel left out (results are then wrong)
};

// Walks the (tile, chunk) stages of this CTA's work items in the order every role uses.
struct StageWalk {
  int w, tile, split, c, c0, c1;
  __device__ __forceinline__ void open(const GemmArgs& a) {
    tile = w / a.splits;
    split = w - tile * a.splits;
    c0 = c = split * a.nchunks / a.splits;
    c1 = (split + 1) * a.nchunks / a.splits;
  }
  __device__ __forceinline__ StageWalk(const GemmArgs& a) : w(blockIdx.x) {
    if (w < a.items) open(a);
  }
  __device__ __forceinline__ bool live(const GemmArgs& a) const { return w < a.items; }
  __device__ __forceinline__ bool last_chunk() const { return c + 1 == c1; }
  // The chunk to load at this step.  The CTAs of a wave walk their K ranges in step; starting each
  // tile at a different chunk keeps them from all asking the L2 for the same activation tile at
  // the same moment.  (The sum over chunks is taken in this order; it is fixed per tile.)
  __device__ __forceinline__ int chunk(const GemmArgs& a) const {
    if (!a.rotate) return c;
    const int len = c1 - c0;
    return c0 + (c - c0 + tile * 5) % len;
  }
  __device__ __forceinline__ void next(const GemmArgs& a) {
    if (++c == c1) {
      w += gridDim.x;
      if (w < a.items) open(a);
    }
  }
};

template <int NC, int P, int FMT>
struct GemmSmem {
  static constexpr int kWBytes = FMT == G_MLX4 ? kMlxWBytes : kFp8WBytes;
  static constexpr int kBBytes = P * NC * 512;                  // 256 K x NC rows of bf16 per piece
  static constexpr int kXBytes = FMT == G_MLX4 ? NC * 16 : 0;   // 4 groups x NC sums
  static constexpr int kStage = kWBytes + kBBytes + kXBytes;
  static __host__ __device__ size_t bytes(int stages) { return (size_t)stages * kStage + 1024 + 512; }
};

// Element order along K inside a 16-element MMA step, as the converters emit it.  A thread of the
// preparation kernel owns 8 consecutive elements (one 16-byte row of a core matrix) and places
// element j of them at position pos8(j).
//   MLX4: a packed word's nibbles j and j+4 share a register (low / high half).
//   FP8:  a word's bytes 0,2 and 1,3 share a register.
template <int FMT>
__host__ __device__ inline int pos8(int j) {
  return FMT == G_MLX4 ? 2 * (j & 3) + (j >> 2) : 4 * (j >> 2) + (((j & 1) << 1) | ((j >> 1) & 1));
}

__device__ __forceinline__ uint32_t bf16_bits_rn(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// ---- activation preparation -----------------------------------------------------------------
// Grid (chunk, 8-row block of the NC columns); block of 256 threads = 8 rows x 32 octets of the
// chunk.  Thread: 8 consecutive elements of one activation row -> one 16-byte core-matrix row per
// piece.  Rows past `batch` are written as zeros.  MLX: the sums of x per 64-element group.
template <int NC, int P, int FMT, bool XBF16>
__global__ void __launch_bounds__(256)
tc_prep_x_kernel(const void* __restrict__ xv, unsigned char* __restrict__ xb, float* __restrict__ xtab, int batch,
                 int in_dim) {
  const int c = blockIdx.x, m = blockIdx.y * 8 + (threadIdx.x >> 5), o = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();  // x may be the output of the kernel in front; the tiles may still be read by it
  float v[8];
  if (m < batch) {
    if (XBF16) {
      const uint4 q = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(xv) + (size_t)m * in_dim + c * kChunkK + o * 8);
      const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[2 * k] = __uint_as_float(ws[k] << 16);
        v[2 * k + 1] = __uint_as_float(ws[k] & 0xFFFF0000u);
      }
    } else {
      const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(xv) + (size_t)m * in_dim + c * kChunkK + o * 8);
      const float4 a = p[0], b = p[1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
      v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
  }
  if (FMT == G_MLX4) {
    float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if ((o & 7) == 0) xtab[((size_t)c * 4 + (o >> 3)) * NC + m] = s;
  }
  // K step = o >> 1, K half = o & 1; the 8 elements fill one core-matrix row of that half
  unsigned char* dst = xb + (size_t)c * (P * NC * 512) + (o >> 1) * (NC * 32) + (o & 1) * ((NC / 8) * 128) + (m >> 3) * 128 +
                       (m & 7) * 16;
#pragma unroll
  for (int p = 0; p < P; ++p) {
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      h[j] = bf16_bits_rn(v[j]);
      v[j] -= __uint_as_float(h[j] << 16);  // exact: the remainder of a round-to-nearest fits f32
    }
    uint32_t e[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) e[pos8<FMT>(j)] = h[j];
    *reinterpret_cast<uint4*>(dst + (size_t)p * (NC * 512)) =
        make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
  }
}

// HC (4, 8 or 16) consecutive accumulator columns of this warp's 32 lanes into registers: the
// load is issued, and waited for separately so that other work can go in between.
template <int HC>
__device__ __forceinline__ void tmem_ld_issue(uint32_t taddr, uint32_t (&t)[HC]) {
  static_assert(HC == 4 || HC == 8 || HC == 16, "4, 8 or 16 columns");
  if constexpr (HC == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(t[0]), "=r"(t[1]), "=r"(t[2]), "=r"(t[3])
                 : "r"(taddr)
                 : "memory");
  } else if constexpr (HC == 8) {
    tmem_ld8(taddr, t);
  } else {
    tmem_ld16(taddr, t);
  }
}
template <int HC>
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&t)[HC]) {
  if constexpr (HC == 4) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]) : : "memory");
  } else {
    tmem_wait_ld(t);
  }
}

// ---- the product kernel -----------------------------------------------------------------------
template <int NC, int P, int FMT>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ GemmArgs a) {
  static_assert(NC == 16 || NC == 32 || NC == 64, "accumulator blocks of 16, 32 or 64 columns");
  typedef GemmSmem<NC, P, FMT> SM;
  constexpr int kWBytes = SM::kWBytes, kBBytes = SM::kBBytes, kXBytes = SM::kXBytes, kStage = SM::kStage;
  constexpr bool kMLX = FMT == G_MLX4;
  constexpr int NA = 2;                                        // A buffers of 128 columns, one per converter group
  // A stage is handed from the MMA warp to the epilogue in two units of 128 elements; a unit is
  // two accumulator blocks of NC columns (one per 64 elements, an MLX group).  Every hand-over
  // costs each side a few hundred cycles of waits, fences and arrivals, so it is not done per block.
  constexpr int UPS = 2;                                       // units per stage
  constexpr int UC = 2 * NC;                                   // accumulator columns of a unit
  constexpr int ND = 256 / UC > 4 ? 4 : 256 / UC;              // units in the accumulator ring
  constexpr int HC = NC / 4;                                   // columns an epilogue warp owns
  constexpr uint32_t kCols = 512;
  static_assert(NA * 128 + ND * UC <= 512, "TMEM plan");
  TP(if (threadIdx.x == 0) atomicMin(&g_tc_span[0], gtime());)
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  const int S = a.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)S * kStage);
  // bars: full[S], empty[S], a_ready[NA], a_free[NA], d_full[ND], d_free[ND], cluster
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 2 * NA + 2 * ND + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* recv = reinterpret_cast<float*>(tmem_holder + 4);  // cluster launches: [split - 1][column m][128] partial sums from the other CTAs

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + S);
  const uint32_t aready0 = smem_u32(bars + 2 * S), afree0 = aready0 + 8 * NA;
  const uint32_t dfull0 = afree0 + 8 * NA, dfree0 = dfull0 + 8 * ND;
  const uint32_t clbar = dfree0 + 8 * ND;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);
      // the converters, the epilogue (MLX: scale data and sums of x), the MMA commits (B tile)
      mbar_init(empty0 + 8 * s, kConvWarps + (kMLX ? kEpiWarps : 0) + kMmaWarps);
    }
    for (int b = 0; b < NA; ++b) {
      mbar_init(aready0 + 8 * b, kConvWarps);
      mbar_init(afree0 + 8 * b, kMmaWarps);
    }
    for (int b = 0; b < ND; ++b) {
      mbar_init(dfull0 + 8 * b, 1);
      mbar_init(dfree0 + 8 * b, kEpiWarps);
    }
    if (a.cluster) mbar_init(clbar, kEpiWarps * (a.splits - 1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kWarpMMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (a.cluster) cluster_sync_all();  // the first CTA's barrier is initialised before any peer can arrive on it
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmemA0 = tmem_base, tmemD0 = tmem_base + NA * 128;
  bool ok = true;
  StageWalk sw(a);
  TP(const bool tr = blockIdx.x == gridDim.x / 2; if (tr && tid == 0) g_tc_trace[7][0] = clock64();)
  TP(if (tid == 0) { const unsigned long long g = gtime(); atomicMax(&g_tc_span[1], g); atomicMin(&g_tc_span[3], g); })

  if (warp == kWarpTMA) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      auto load_w = [&](int slot, const StageWalk& s) {
        bulk_load_1d(smem_u32(ring + (size_t)slot * kStage), a.w + ((size_t)s.tile * a.nchunks + s.chunk(a)) * kWBytes, kWBytes,
                     full0 + 8 * slot);
      };
      auto load_x = [&](int slot, const StageWalk& s) {
        const uint32_t dst = smem_u32(ring + (size_t)slot * kStage) + kWBytes;
        const int c = s.chunk(a);
        if (DBG(2)) return;  // tuning: no activation traffic
        bulk_load_1d(dst, a.xb + (size_t)c * kBBytes, kBBytes, full0 + 8 * slot);
        if (kMLX) bulk_load_1d(dst + kBBytes, a.xtab + (size_t)c * (4 * NC), kXBytes, full0 + 8 * slot);
      };
      // The weights do not depend on the kernel in front: fill the ring with them first, then wait
      // for the prepared activations and add the B tiles of those stages.
      // (Only the first two stages at once: a grid that asked for all its rings at the same moment
      // would see every CTA's first stage land last.  The rest follows when the first stage is in.)
      int i = 0;
      StageWalk sw0 = sw;
      for (; i < S && i < 2 && sw0.live(a); ++i, sw0.next(a)) {
        mbar_expect_tx(full0 + 8 * i, DBG(2) ? kWBytes : kStage);
        load_w(i, sw0);
      }
      pdl_wait();
      TP(if (tr) g_tc_trace[7][2] = clock64();)
      for (int j = 0; j < i; ++j, sw.next(a)) {
        load_x(j, sw);
        TP(if (tr && j < 64) g_tc_trace[0][j] = clock64();)
      }
      for (; sw.live(a) && ok; ++i, sw.next(a)) {
        const int slot = i % S, round = i / S;
        if (round > 0) ok = mbar_wait(empty0 + 8 * slot, (round - 1) & 1, a.status, 301);
        else if (i == 2) ok = mbar_wait(full0, 0, a.status, 309);
        if (!ok) break;
        mbar_expect_tx(full0 + 8 * slot, DBG(2) ? kWBytes : kStage);
        load_w(slot, sw);
        load_x(slot, sw);
        TP(if (tr && i < 64) g_tc_trace[0][i] = clock64();)
      }
    }
  } else if (warp == kWarpMMA) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the stages and waits; one elected lane issues.  (Everything the
    // instructions need is the same in all lanes, which lets it live in uniform registers.)
    // instruction descriptor: D f32, A bf16, B bf16, both K-major, N = NC, M = 128
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NC >> 3) << 17) | ((128u >> 4) << 24);
    constexpr uint32_t kLBO = (NC / 8) * 128, kSBO = 128;  // K-adjacent / N-adjacent core matrices
    const uint64_t desc_hi = ((uint64_t)(kLBO >> 4) << 16) | ((uint64_t)(kSBO >> 4) << 32) | (1ull << 46);
    int du = 0;  // units handed to the epilogue so far
    for (int i = 0; sw.live(a) && ok; ++i) {
      const int slot = i % S, ab = i % NA;
      ok = mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 302);
      if (ok) ok = mbar_wait(aready0 + 8 * ab, (i / NA) & 1, a.status, 303);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      TP(if (tr && lane == 0 && i < 64) g_tc_trace[1][i] = clock64();)
      const uint32_t bbase = smem_u32(ring + (size_t)slot * kStage) + kWBytes;
      const uint32_t acol = tmemA0 + ab * 128;
#pragma unroll
      for (int u = 0; u < UPS; ++u, ++du) {
        const int ds = du % ND;
        if (du >= ND) {
          ok = __all_sync(0xffffffffu, mbar_wait(dfree0 + 8 * ds, (du / ND - 1) & 1, a.status, 304));
          if (!ok) break;
          tc_fence_after();
        }
        if (elect_one()) {
          if (!DBG(4)) {
#pragma unroll
            for (int p = 0; p < P; ++p) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {  // K steps 8u .. 8u+7: the first four into block 0, the others into block 1
                const int ks = 8 * u + k;
                const uint64_t bdesc = desc_hi | (uint64_t)(((bbase + p * (NC * 512) + ks * (NC * 32)) >> 4) & 0x3FFF);
                umma_bf16_ts(tmemD0 + ds * UC + (k >> 2) * NC, acol + ks * 8, bdesc, idesc, (p | (k & 3)) != 0);
              }
            }
          }
          umma_commit(dfull0 + 8 * ds);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (elect_one()) {
        umma_commit(afree0 + 8 * ab);
        umma_commit(empty0 + 8 * slot);
      }
      __syncwarp();
      TP(if (tr && lane == 0 && i < 64) g_tc_trace[2][i] = clock64();)
      sw.next(a);
    }
  } else if (warp < kConvWarps) {
    // ------------------------------------------------------------------ converters
    // All eight warps convert every stage, into the A buffer of the stage's parity (the MMAs of one
    // stage read one buffer while the next stage is written into the other).  Thread = row r of
    // the tile and one half of the stage's K range.
    const int q4 = warp & 3, kh = warp >> 2;
    const int r = q4 * 32 + lane;
    for (int i = 0; sw.live(a) && ok; ++i, sw.next(a)) {
      const int slot = i % S, ab = i & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 305));
      if (ok && i >= NA) ok = __all_sync(0xffffffffu, mbar_wait(afree0 + 8 * ab, ((i / NA) - 1) & 1, a.status, 306));
      if (!ok) break;
      tc_fence_after();
      TP(if (tr && warp == 0 && lane == 0 && i < 64) g_tc_trace[3][i] = clock64();)
      const unsigned char* st = ring + (size_t)slot * kStage;
      const uint32_t abuf = tmemA0 + ((uint32_t)(q4 * 32) << 16) + ab * 128 + kh * 64;
      if (DBG(8)) {  // tuning: nothing converted
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(aready0 + 8 * ab);
          mbar_arrive(empty0 + 8 * slot);
        }
        continue;
      }
      if (kMLX) {
        // 128 nibbles of the row -> 128 bf16 (16 + n) -> 64 TMEM columns
        uint4 qv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) qv[u] = *reinterpret_cast<const uint4*>(st + r * 128 + (((4 * kh + u) ^ (r & 7)) << 4));
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t ws[4] = {qv[u].x, qv[u].y, qv[u].z, qv[u].w};
#pragma unroll
          for (int s2 = 0; s2 < 2; ++s2) {  // a K = 16 step is two packed words
            uint32_t regs[8];
#pragma unroll
            for (int wi = 0; wi < 2; ++wi) {
              const uint32_t w = ws[2 * s2 + wi];
              regs[4 * wi + 0] = ((w << 3) & 0x00780078u) | 0x41804180u;  // nibbles 0 and 4
              regs[4 * wi + 1] = ((w >> 1) & 0x00780078u) | 0x41804180u;  // nibbles 1 and 5
              regs[4 * wi + 2] = ((w >> 5) & 0x00780078u) | 0x41804180u;  // nibbles 2 and 6
              regs[4 * wi + 3] = ((w >> 9) & 0x00780078u) | 0x41804180u;  // nibbles 3 and 7
            }
            tmem_st8(abuf + (2 * u + s2) * 8, regs);
          }
        }
      } else {
        // 128 E4M3 bytes of the row -> 128 bf16 -> 64 TMEM columns, four 16-byte units at a time
#pragma unroll
        for (int ub = 0; ub < 8; ub += 4) {
          uint4 qv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            // 16-byte unit U of row r in the block of K-major core matrices (see fp8_mma.cu):
            // [K step U / 2][half U % 2][row group r / 8][row r % 8]; a warp's 32 rows read 512 contiguous bytes
            const int U = 8 * kh + ub + u;
            qv[u] = *reinterpret_cast<const uint4*>(st + (U >> 1) * 4096 + (U & 1) * 2048 + (r >> 3) * 128 + (r & 7) * 16);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint32_t ws[4] = {qv[u].x, qv[u].y, qv[u].z, qv[u].w};
            uint32_t regs[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t w = ws[k];
              // bytes 0,2 / 1,3: sign to bit 15, exponent and mantissa to bits 10..4, times 2^120
              const uint32_t a02 = ((w << 4) & 0x07F007F0u) | ((w << 8) & 0x80008000u);
              const uint32_t a13 = ((w >> 4) & 0x07F007F0u) | (w & 0x80008000u);
              asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(regs[2 * k]) : "r"(a02), "r"(0x7B807B80u));
              asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(regs[2 * k + 1]) : "r"(a13), "r"(0x7B807B80u));
            }
            tmem_st8(abuf + (ub + u) * 8, regs);
          }
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(aready0 + 8 * ab);
        mbar_arrive(empty0 + 8 * slot);
      }
      TP(if (tr && warp == 0 && lane == 0 && i < 64) g_tc_trace[4][i] = clock64();)
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // Warp (q4, cq): rows 32 q4 .. +31 of the tile, columns cq * HC .. + HC - 1 of every block.
    const int q4 = warp & 3, cq = (warp - kConvWarps) >> 2;
    const int r = q4 * 32 + lane;
    const int et = tid - kConvWarps * 32;
    const uint32_t dbase = tmemD0 + ((uint32_t)(q4 * 32) << 16) + cq * HC;
    const int mcols = a.batch - cq * HC;  // columns of this warp that hold activation rows
    float2 acc[HC / 2];
#pragma unroll
    for (int j = 0; j < HC / 2; ++j) acc[j] = make_float2(0.f, 0.f);
    int du = 0;
    for (int i = 0; sw.live(a) && ok; ++i) {
      const int slot = i % S;
      const unsigned char* st = ring + (size_t)slot * kStage;
      uint32_t meta[4] = {0, 0, 0, 0};
      if (kMLX) {
        ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 307));
        if (!ok) break;
        const uint4 mv = *reinterpret_cast<const uint4*>(st + kTileRows * 128 + r * 16);
        meta[0] = mv.x, meta[1] = mv.y, meta[2] = mv.z, meta[3] = mv.w;
      }
      const float* xs = reinterpret_cast<const float*>(st + kWBytes + kBBytes) + cq * HC;
#pragma unroll
      for (int u = 0; u < UPS; ++u, ++du) {
        const int ds = du % ND;
        ok = __all_sync(0xffffffffu, mbar_wait(dfull0 + 8 * ds, (du / ND) & 1, a.status, 308));
        if (!ok) break;
        tc_fence_after();
        TP(if (tr && et == 0 && u == 0 && i < 64) g_tc_trace[5][i] = clock64();)
        uint32_t t[2][HC];  // this warp's columns of the unit's two blocks, both loads in flight together
        tmem_ld_issue<HC>(dbase + ds * UC, t[0]);
        tmem_ld_issue<HC>(dbase + ds * UC + NC, t[1]);
        tmem_ld_wait<HC>(t[0]);
        tmem_ld_wait<HC>(t[1]);
        tc_fence_before();
        warp_arrive(dfree0 + 8 * ds, lane);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int g = 2 * u + b;  // 64-element group of the stage
          if (kMLX) {
            const float sc = __uint_as_float(meta[g] << 16), bi = __uint_as_float(meta[g] & 0xFFFF0000u);
            const float b16 = fmaf(-16.f, sc, bi);  // the 16 added to every nibble comes out through sum x
            const float2 sc2 = make_float2(sc, sc), bi2 = make_float2(b16, b16);
#pragma unroll
            for (int j = 0; j < HC / 4; ++j) {
              if (4 * j < mcols) {
                const float4 xv = *reinterpret_cast<const float4*>(xs + g * NC + 4 * j);
                fma2(acc[2 * j], sc2, make_float2(__uint_as_float(t[b][4 * j]), __uint_as_float(t[b][4 * j + 1])));
                fma2(acc[2 * j + 1], sc2, make_float2(__uint_as_float(t[b][4 * j + 2]), __uint_as_float(t[b][4 * j + 3])));
                fma2(acc[2 * j], bi2, make_float2(xv.x, xv.y));
                fma2(acc[2 * j + 1], bi2, make_float2(xv.z, xv.w));
              }
            }
          } else {
            // FP8: the tensor core sums 64 elements per block; the blocks are added here in f32
#pragma unroll
            for (int j = 0; j < HC / 2; ++j) {
              acc[j].x += __uint_as_float(t[b][2 * j]);
              acc[j].y += __uint_as_float(t[b][2 * j + 1]);
            }
          }
        }
      }
      if (!ok) break;
      if (kMLX) warp_arrive(empty0 + 8 * slot, lane);  // scale data and sums of x are no longer needed
      TP(if (tr && et == 0 && i < 64) g_tc_trace[6][i] = clock64();)
      const bool item_done = sw.last_chunk();
      const int tile = sw.tile, split = sw.split;
      sw.next(a);
      if (!item_done) continue;
      // ---- the item is complete ----
      const int row = tile * kTileRows + r;
      float rs = 1.f, rb = 0.f;
      if (!kMLX && row < a.out_dim) {
        rs = a.scale[row];
        if (a.bias) rb = a.bias[row];
      }
      auto finish = [&](float v) { return kMLX ? v : (a.bias ? __fadd_rn(__fmul_rn(v, rs), rb) : __fmul_rn(v, rs)); };
      if (NC <= 32 && a.cluster) {  // (64 columns never fit the receive area: no such code, and no registers for it, in that kernel)
        // The K splits of this tile are the CTAs of this cluster (rank == split), one item each: ranks
        // above 0 put their sums into rank 0's shared memory and arrive on its barrier (one releasing
        // arrival per warp); rank 0 waits, adds in split order (the scratch path's order) and stores.
        if (split != 0) {
#pragma unroll
          for (int j = 0; j < HC / 2; ++j) {
            const int m = cq * HC + 2 * j;
            cluster_store_f32(cluster_map(smem_u32(recv + ((size_t)(split - 1) * NC + m) * kTileRows + r), 0), acc[j].x);
            cluster_store_f32(cluster_map(smem_u32(recv + ((size_t)(split - 1) * NC + m + 1) * kTileRows + r), 0), acc[j].y);
          }
          __syncwarp();
          if (lane == 0) cluster_arrive_release(cluster_map(clbar, 0));
        } else {
          ok = __all_sync(0xffffffffu, mbar_wait_cluster(clbar, 0, a.status, 310));
          if (ok) {
#pragma unroll
            for (int j = 0; j < HC / 2; ++j) {
              const int m = cq * HC + 2 * j;
              float s0 = acc[j].x, s1 = acc[j].y;
              for (int s2 = 1; s2 < a.splits; ++s2) {
                s0 += recv[((size_t)(s2 - 1) * NC + m) * kTileRows + r];
                s1 += recv[((size_t)(s2 - 1) * NC + m + 1) * kTileRows + r];
              }
              if (row < a.out_dim) {
                if (m < a.batch) a.out[(size_t)m * a.out_dim + row] = finish(s0);
                if (m + 1 < a.batch) a.out[(size_t)(m + 1) * a.out_dim + row] = finish(s1);
              }
            }
          }
        }
#pragma unroll
        for (int j = 0; j < HC / 2; ++j) acc[j] = make_float2(0.f, 0.f);
      } else if (a.splits == 1) {
#pragma unroll
        for (int j = 0; j < HC / 2; ++j) {
          const int m = cq * HC + 2 * j;
          if (row < a.out_dim) {
            if (m < a.batch) a.out[(size_t)m * a.out_dim + row] = finish(acc[j].x);
            if (m + 1 < a.batch) a.out[(size_t)(m + 1) * a.out_dim + row] = finish(acc[j].y);
          }
          acc[j] = make_float2(0.f, 0.f);
        }
      } else {
        // Partial sums of this K range go to scratch; the CTA that arrives last at the tile adds the
        // partials in split order (so the result does not depend on arrival order) and stores.
        float* part = a.scratch + ((size_t)tile * a.splits + split) * (NC * kTileRows);
#pragma unroll
        for (int j = 0; j < HC / 2; ++j) {
          const int m = cq * HC + 2 * j;
          if (m < a.batch) part[m * kTileRows + r] = acc[j].x;
          if (m + 1 < a.batch) part[(m + 1) * kTileRows + r] = acc[j].y;
          acc[j] = make_float2(0.f, 0.f);
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (et == 0) *last_flag = (atomicAdd(a.counters + tile, 1u) == (unsigned)a.splits - 1) ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (*last_flag) {
          __threadfence();
          const float* base = a.scratch + (size_t)tile * a.splits * (NC * kTileRows);
          // four columns at a time: a split's four loads are independent and in flight together (one
          // chain of dependent L2 loads per column cost microseconds), without the registers that
          // all HC columns at once would take from the main loop
          constexpr int SB = HC < 4 ? HC : 4;
#pragma unroll 1
          for (int j0 = 0; j0 < HC; j0 += SB) {
            float sum[SB];
#pragma unroll
            for (int j = 0; j < SB; ++j) sum[j] = 0.f;
            for (int s2 = 0; s2 < a.splits; ++s2) {
#pragma unroll
              for (int j = 0; j < SB; ++j) sum[j] += __ldcg(base + (size_t)s2 * (NC * kTileRows) + (cq * HC + j0 + j) * kTileRows + r);
            }
#pragma unroll
            for (int j = 0; j < SB; ++j) {
              const int m = cq * HC + j0 + j;
              if (m < a.batch && row < a.out_dim) a.out[(size_t)m * a.out_dim + row] = finish(sum[j]);
            }
          }
          if (et == 0) a.counters[tile] = 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      }
    }
  }
  TP(if (tr && tid == 0) g_tc_trace[7][1] = clock64();)
  TP(if (tid == 0) atomicMax(&g_tc_span[2], gtime());)
  // ---- wind down: everyone meets, outstanding copies are drained, TMEM is returned ----
  tc_fence_before();
  __syncthreads();
  if (warp == kWarpTMA && lane == 0 && *reinterpret_cast<volatile int*>(a.status) != 0) {
    // a waiter gave up: copies may still be in flight; give each ring slot a bounded chance to land
    for (int s = 0; s < S; ++s) {
      long long t0 = clock64();
      while (!mbar_try_wait(full0 + 8 * s, 0) && !mbar_try_wait(full0 + 8 * s, 1) && clock64() - t0 < kTimeoutCycles / 8) {
      }
    }
  }
  __syncthreads();
  if (warp == kWarpMMA) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kCols) : "memory");
  }
}

// ---- host side --------------------------------------------------------------------------------

constexpr int kMaxIn = 65536;
constexpr size_t kXbBytes = (size_t)128 * kMaxIn;          // 64 columns x 1 piece or 16 x 3, 2 bytes each
constexpr size_t kXtabFloats = (size_t)kMaxIn;             // (in/64) groups x 64 columns
constexpr int kMaxItems = 320;                             // (tile, split) items with partial sums at once
constexpr size_t kScratchFloats = (size_t)kMaxItems * kTileRows * 64;
constexpr size_t kMaxCounters = 4096;
constexpr size_t kSmemBudget2 = 222 * 1024;

struct GemmBufs {
  unsigned char* xb = nullptr;
  float* xtab = nullptr;
  int* status = nullptr;
  float* scratch = nullptr;
  unsigned int* counters = nullptr;
};

// Allocated on a device's first small-batch product; published only when complete.
GemmBufs* gemm_bufs(int device, bool allocate = true) {
  static GemmBufs bufs[kMaxDevices];
  static bool ready[kMaxDevices] = {};
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (ready[device]) return &bufs[device];
  if (!allocate) return nullptr;
  GemmBufs b;
  bool ok = cudaMalloc(&b.xb, kXbBytes) == cudaSuccess && cudaMalloc(&b.xtab, kXtabFloats * 4) == cudaSuccess &&
            cudaMalloc(&b.status, 256) == cudaSuccess && cudaMalloc(&b.scratch, kScratchFloats * 4) == cudaSuccess &&
            cudaMalloc(&b.counters, kMaxCounters * 4) == cudaSuccess;
  ok = ok && cudaMemset(b.status, 0, 256) == cudaSuccess && cudaMemset(b.counters, 0, kMaxCounters * 4) == cudaSuccess &&
       cudaDeviceSynchronize() == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    cudaFree(b.xb);
    cudaFree(b.xtab);
    cudaFree(b.status);
    cudaFree(b.scratch);
    cudaFree(b.counters);
    return nullptr;
  }
  bufs[device] = b;
  ready[device] = true;
  return &bufs[device];
}

}  // namespace

// K splits per tile: the split whose busiest CTA spends the least time (items are dealt to the
// CTAs round-robin), in units of one stage; fix_cost is what writing and re-reading one item's
// partial sums costs in those units.
int tc_choose_splits(int ntiles, int nchunks, int sms, int max_items, float fix_cost) {
  int best = 1;
  float best_cost = -1.f;
  for (int s = 1; s <= 8 && s <= nchunks; ++s) {
    const long items = (long)ntiles * s;
    if (items > max_items && s > 1) break;
    const int grid = items < sms ? (int)items : sms;
    const long per_cta = (items + grid - 1) / grid;
    const float cost = per_cta * ((nchunks + s - 1) / s + (s > 1 ? fix_cost : 0.f));
    if (best_cost < 0.f || cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

namespace {

int g_rotate = 1;  // see StageWalk::chunk
int g_dbg = 0;     // tuning build only

struct GemmDesc {
  const unsigned char* tiled;
  const float* scale;
  const float* bias;
  int device, out_dim, in_dim;
};

template <int NC, int P, int FMT, bool XBF16>
int launch_pass(const GemmDesc& w, float* out, const void* x, int nb, GemmBufs* bufs, cudaStream_t stream) {
  typedef GemmSmem<NC, P, FMT> SM;
  DeviceState& st = device_state(w.device);
  GemmArgs a;
  memset(&a, 0, sizeof a);
  a.w = w.tiled;
  a.xb = bufs->xb;
  a.xtab = bufs->xtab;
  a.scale = w.scale;
  a.bias = w.bias;
  a.out = out;
  a.status = bufs->status;
  a.scratch = bufs->scratch;
  a.counters = bufs->counters;
  a.out_dim = w.out_dim;
  a.in_dim = w.in_dim;
  a.batch = nb;
  a.ntiles = (w.out_dim + kTileRows - 1) / kTileRows;
  a.nchunks = w.in_dim / kChunkK;
  int max_items = (int)(kScratchFloats / ((size_t)NC * kTileRows));
  if (a.ntiles > (int)kMaxCounters) max_items = 0;
  a.splits = options().mlx_splits > 0 ? (options().mlx_splits < a.nchunks ? options().mlx_splits : a.nchunks)
                                      : tc_choose_splits(a.ntiles, a.nchunks, st.sm_count, max_items, NC / 32.f);
  while (a.splits > 1 && (long)a.ntiles * a.splits > max_items) --a.splits;
  a.items = a.ntiles * a.splits;
  const int grid = a.items < st.sm_count ? a.items : st.sm_count;
  constexpr size_t kRecvBytes = 16 * 1024;
  const bool want_cluster = options().mlx_cluster && a.splits > 1 && a.splits <= 8 && a.items == grid &&
                            (size_t)(a.splits - 1) * NC * kTileRows * 4 <= kRecvBytes;
  const size_t extra = want_cluster ? kRecvBytes : 0;
  int stages = (int)((kSmemBudget2 - SM::bytes(0) - extra) / SM::kStage);
  if (stages > 8) stages = 8;
  if (stages < 2) return fail(GOPH_E_UNSUPPORTED, "small-batch tensor-core path: a stage of %d bytes leaves no room for a ring", SM::kStage);
  a.stages = stages;
  a.rotate = g_rotate;
  a.dbg = g_dbg;
  size_t smem = SM::bytes(stages) + extra;
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM (the kernel owns all of TMEM)

  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(a.nchunks, NC / 8);
  cfg.blockDim = dim3(256);
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, tc_prep_x_kernel<NC, P, FMT, XBF16>, x, bufs->xb, bufs->xtab, nb, w.in_dim));
  auto kern = tc_gemm_kernel<NC, P, FMT>;
  GOPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  if (want_cluster) {
    // only when the device holds every cluster of the grid at once (asked once per kernel, split count and device)
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = a.splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
    static std::mutex mu;
    static int room[kMaxDevices][9];
    static bool known[kMaxDevices][9] = {};
    int resident;
    {
      std::lock_guard<std::mutex> lock(mu);
      if (!known[w.device][a.splits]) {
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
          cudaGetLastError();
          n = 0;
        }
        room[w.device][a.splits] = n;
        known[w.device][a.splits] = true;
      }
      resident = room[w.device][a.splits];
    }
    if (resident * a.splits >= grid) a.cluster = 1;
    else cfg.numAttrs = 1;
  }
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  return GOPH_OK;
}

// Passes of up to 64 rows (bf16 activations, one piece) or 16 rows (f32 activations, three pieces).
template <int FMT>
int run_passes(const GemmDesc& w, float* out, const void* x, bool x_bf16, int batch, cudaStream_t stream) {
  if (w.in_dim % kChunkK != 0 || w.in_dim > kMaxIn)
    return fail(GOPH_E_UNSUPPORTED, "small-batch tensor-core path: in_dim=%d is not a multiple of 256 up to %d", w.in_dim, kMaxIn);
  if ((uintptr_t)x % 16) return fail(GOPH_E_INVALID, "x must be 16-byte aligned");
  GemmBufs* bufs = gemm_bufs(w.device);
  if (!bufs) return fail(GOPH_E_NOMEM, "cannot allocate the small-batch tensor-core path's device scratch");
  const int cap = x_bf16 ? 64 : 16;
  const size_t xstride = (size_t)w.in_dim * (x_bf16 ? 2 : 4);
  for (int b0 = 0; b0 < batch;) {
    const int nb = batch - b0 < cap ? batch - b0 : cap;
    const void* xp = static_cast<const unsigned char*>(x) + (size_t)b0 * xstride;
    float* op = out + (size_t)b0 * w.out_dim;
    int rc;
    if (!x_bf16) rc = launch_pass<16, 3, FMT, false>(w, op, xp, nb, bufs, stream);
    else if (nb <= 16) rc = launch_pass<16, 1, FMT, true>(w, op, xp, nb, bufs, stream);
    else if (nb <= 32) rc = launch_pass<32, 1, FMT, true>(w, op, xp, nb, bufs, stream);
    else rc = launch_pass<64, 1, FMT, true>(w, op, xp, nb, bufs, stream);
    if (rc) return rc;
    b0 += nb;
  }
  return GOPH_OK;
}

}  // namespace

int tc_gemm_fp8_converted(const goph_fp8_linear* w, float* out, const void* x, bool x_bf16, int batch, cudaStream_t stream) {
  if (!w->tiled) return fail(GOPH_E_UNSUPPORTED, "FP8 linear is not in the tensor-core layout");
  GemmDesc d{w->tiled, w->scale, w->bias, w->device, w->out_dim, w->in_dim};
  return run_passes<G_FP8>(d, out, x, x_bf16, batch, stream);
}

int tc_gemm_mlx(const goph_mlx_weight* w, float* out, const void* x, bool x_bf16, int batch, cudaStream_t stream) {
  if (!w->tiled) return fail(GOPH_E_UNSUPPORTED, "weight is not in the tiled layout");
  GemmDesc d{w->tiled, nullptr, nullptr, w->device, w->out_dim, w->in_dim};
  return run_passes<G_MLX4>(d, out, x, x_bf16, batch, stream);
}

#ifdef GOPH_TUNING
void tc_gemm_tuning_set(int dbg, int rotate) {
  g_dbg = dbg;
  g_rotate = rotate;
}
int tc_gemm_span(unsigned long long* out4, int reset) {
  if (reset) {
    const unsigned long long init[4] = {~0ull, 0ull, 0ull, ~0ull};
    return cudaMemcpyToSymbol(g_tc_span, init, sizeof init) == cudaSuccess ? 0 : -1;
  }
  return cudaMemcpyFromSymbol(out4, g_tc_span, 4 * sizeof(unsigned long long)) == cudaSuccess ? 0 : -1;
}
int tc_gemm_probe(long long* out64) {
  return cudaMemcpyFromSymbol(out64, g_tc_trace, 8 * 64 * sizeof(long long)) == cudaSuccess ? 0 : -1;
}
#endif

void tc_gemm_status_clear(int device) {
  GemmBufs* b = gemm_bufs(device, false);
  if (b) cudaMemset(b->status, 0, sizeof(int));
}

int tc_gemm_status(int device) {
  GemmBufs* b = gemm_bufs(device, false);
  if (!b) return 0;  // no small-batch product has run on this device
  int v = -1;
  cudaMemcpy(&v, b->status, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

}  // namespace goph

#ifdef GOPH_TUNING
GOPH_API int goph_tuning_probe(long long* out64) { return goph::tc_gemm_probe(out64); }
GOPH_API int goph_tuning_span(unsigned long long* out4, int reset) { return goph::tc_gemm_span(out4, reset); }
GOPH_API int goph_tuning_set(int dbg, int rotate) {
  goph::tc_gemm_tuning_set(dbg, rotate);
  return 0;
}
#endif
