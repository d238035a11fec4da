// MLX 4-bit weights on the 5th-generation tensor cores (tcgen05 + TMEM), integer arithmetic.
//
// Why a GEMV goes to the tensor pipe: at B200's HBM rate one SM has to consume ~47 nibbles
// per clock, and its integer/logic pipe issues 64 lane-ops per clock.  Any formulation that
// turns each nibble into a float on the CUDA cores needs at least one logic op per nibble plus
// the FMA and cannot reach the HBM roofline.  Here the nibbles stay integers: three logic ops
// turn a packed word into eight unsigned bytes, the tensor cores multiply them (kind::i8, exact
// int32 accumulation), and the CUDA cores only apply the per-group scales.
//
// Arithmetic
//   * A operand (weights): nibble n as the unsigned byte n.
//   * B operand (activations): each 64-element group of an activation row is put on a common
//     power-of-two scale 2^(E-26), E the exponent of the group's largest magnitude, and every
//     element becomes the integer q = round(x * 2^(26-E)), |q| <= 2^26 — at least as fine as
//     the f32 spacing of the group's largest elements.  q is written as four balanced base-128
//     digits, one signed-byte B row per digit (three digits is an option for bf16-valued x).
//   * One int32 accumulator block per 64-element group: D_j[row] = sum_k n_k * digit_j(q_k),
//     exact.  The epilogue rebuilds sum_k n_k q_k = (D0 + 128 D1) + 16384 (D2 + 128 D3) (two
//     exact integers, one fused multiply-add), scales by 2^(E-26) and forms
//     s_g * dot + b_g * sum(x)  in f32 — mlx.GemvTo's expression (backends/mlx/gemv.go:178-209).
//
// Pipeline of one CTA (18 warps; persistent over
// (128-row tile, K range) items; a stage is one 256-element chunk of the tile, or two chunks for
// the nibble formats when tensor memory has the columns):
//   TMA producer warp: one bulk copy per stage of the weight's blocks (the tiled layout stores
//     exactly the shared-memory image of a stage, so every copy is one sequential burst) into a
//     ring of up to 8 stages guarded by full/empty mbarriers, and one of the stage's B tiles
//     (the digits of x, laid out for the tensor core by mlx_prep_x_kernel in front of this
//     kernel, or by this CTA itself for short K ranges).  The first two stages are asked for at
//     once, the rest of the ring when the first has landed.
//   8 converter warps in two groups that take alternate stages, thread = row of the tile:
//     swizzled LDS.128 -> bytes -> tcgen05.st into a ring of A buffers in TMEM (two to four
//     deep, as the 512 columns allow).  Both groups follow every stage's barriers.
//   MMA warp: waits as a warp, one elected lane issues 8 tcgen05.mma (M128 x N x K32, A from
//     TMEM, B straight from the stage) per chunk and commits to the accumulators', the A
//     buffer's and the stage's mbarriers.  Q8_0 reads A from the stage as it lies (no converters).
//   Epilogue warps, two per TMEM lane quarter, each with its share of a
//     stage's accumulator blocks: tcgen05.ld, scales, running sums in registers; at the end of
//     an item the parts are added through shared memory and either stored, or (K split) written
//     to scratch, where the CTA that arrives last adds them in split order (result independent
//     of arrival order).
// Every wait is bounded (~2 s): a waiter that gives up records a code in the status word and
// the CTA winds down (copies drained, TMEM returned) instead of spinning.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <tuple>

#include "goph_internal.cuh"
#include "mlx_mma.cuh"
#include "tc_common.cuh"

namespace goph {

using namespace tc;

namespace {

// Tuning build only (-DGOPH_TUNING): one CTA in the middle of the grid records clock64 at the
// hand-over points of its first 64 stages; goph_tuning_probe_gemv copies the timeline out.
#ifdef GOPH_TUNING
__device__ long long g_mma_trace[8][64];
#define TP(...) __VA_ARGS__
#define DBG(bit) (a.dbg & (bit))  // parts of the kernel left out (results are then wrong)
#else
#define TP(...)
#define DBG(bit) 0
#endif

constexpr int kTileRows = 128;
constexpr int kChunkK = 256;                  // elements per pipeline stage
constexpr int kStageMBytes = kTileRows * 16;  // 16 bytes of scales per row and stage (32 for Q6_K, see Fmt)

// What differs between the weight formats that share this kernel.  A stage is 128 rows x 256
// elements: the weights as the shared-memory image the tensor core (or the converters) want,
// then 16 bytes of scale data per row.
//   MLX4  128 B of nibbles per row (16-byte units XOR-swizzled by row); {scale,bias} bf16 pairs of
//         the 4 groups of 64.  One accumulator block per group (two K=32 MMAs accumulate).
//   Q4K   the same nibble image (one 256-element super-block per row and stage); f16 d, f16 dmin and
//         8 x 12 bits (sc | m << 6).  One accumulator block per 32-element sub-block.
//   Q80   256 signed bytes per row, stored as K-major 8x16-byte core matrices
//         [K step][K half][row group][row][16 B] so the MMA reads them from shared memory as they
//         lie — no conversion at all; 8 f16 block scales.  One accumulator block per 32-element block.
//   Q5K   the 5-bit values written out as 256 unsigned bytes per row at upload (1 byte per weight
//         on the device instead of 0.69: the price of the tensor-core path), in Q80's order; the
//         Q4_K header {d, dmin, 8 x (sc | m << 6)}.  One accumulator block per 32-element sub-block.
//   Q6K   the 6-bit values minus 32 as 256 signed bytes per row (1 byte per weight instead of
//         0.82), in Q80's order; 16 int8 scales + f16 d per row (32 bytes with padding).  One block
//         per K step of 32, whose two 16-element scale groups keep their sums apart like Q4_K's
//         sub-block pairs: the digits of the step's first 16 positions stand in B rows [0, N/2),
//         those of the last 16 in [N/2, N).
enum { FMT_MLX4 = 0, FMT_Q4K = 1, FMT_Q80 = 2, FMT_Q5K = 3, FMT_Q6K = 4 };
template <int FMT>
struct Fmt {
  static constexpr bool kConv = FMT == FMT_MLX4 || FMT == FMT_Q4K;  // nibbles -> bytes through TMEM; else the MMA reads the stage's bytes
  static constexpr bool kHalves = FMT == FMT_Q4K || FMT == FMT_Q6K;  // two scale groups per accumulator block, in the two halves of its columns
  // accumulator blocks per 256-element chunk.  Q4_K: one block per PAIR of 32-element sub-blocks;
  // the two sub-blocks keep their sums apart inside the block because the activation digits of
  // the even sub-block stand in the first half of the B rows (zeros in the odd K steps) and those
  // of the odd sub-block in the second half: accumulator columns [0, N/2) and [N/2, N)
  static constexpr int kBlocks = kConv ? 4 : 8;
  static constexpr int kGroup = FMT == FMT_MLX4 ? 64 : 32;      // elements per entry of the activation tables
  static constexpr int kStageWBytes = kTileRows * (kConv ? 128 : 256);
  static constexpr int kMetaRow = FMT == FMT_Q6K ? 32 : 16;     // bytes of scales per row and stage
  static constexpr int kStageBytes = kStageWBytes + kTileRows * kMetaRow;  // the B tile follows
};
constexpr int kStageWBytes = Fmt<FMT_MLX4>::kStageWBytes;
constexpr int kStageBytes = Fmt<FMT_MLX4>::kStageBytes;

constexpr int kConvWarps = 8;
constexpr int kConvThreads = kConvWarps * 32;
constexpr int kMmaWarps = 1;  // the whole warp walks the stages, one elected lane issues
// Epilogue warps per TMEM lane quarter; each takes an equal part of a stage's accumulator blocks.
// Two for every format.  (Four were tried for Q4_K, whose epilogue is the slowest role of its
// pipeline, 1300 cycles of arithmetic a stage against 500 for MLX: the eight extra warps made every
// role slower and the LM-head product went from 66 to 74 us.)
template <int N, int FMT>
__host__ __device__ constexpr int epi_parts() {
  return 2;
}
template <int N, int FMT>
__host__ __device__ constexpr int mma_threads() {
  return (kConvWarps + 4 * epi_parts<N, FMT>() + 1 + kMmaWarps) * 32;
}
// Stages whose copies are issued at once when a CTA starts.  If every CTA of the grid asked for its
// whole ring at that moment (tens of MB), the memory system would serve those requests interleaved
// and the first stage of every CTA would land last, microseconds late; the rest of the ring is
// asked for when the first stage has arrived.
constexpr int kFirstStages = 2;
constexpr int kThreads = mma_threads<8, FMT_MLX4>();  // of the instantiation the allocation-free entry point launches


}  // namespace

struct MmaArgs {
  const unsigned char* w;  // tiled weight blocks [tile][chunk]
  const float* x;          // [batch][in_dim]
  const unsigned char* xb; // prepared B operand: [chunk][N rows x 256 bytes], canonical K-major core matrices
  const float* xtab;       // prepared tables: [batch][groups] sum of x, then [batch][groups] 2^(E-QBITS)
  float* out;              // [batch][out_dim]
  int* status;             // device word: 0 ok, otherwise the first wait that gave up
  float* scratch;          // split-K partial sums [item][batch][128]
  unsigned int* counters;  // per-tile arrival counters, zero between launches
  int out_dim, in_dim;
  int batch;               // activation rows of this launch (<= MB of the instantiation)
  int ntiles;              // ceil(out_dim / 128)
  int nchunks;             // in_dim / 256
  int splits;              // CTAs sharing the K range of one tile
  int items;               // ntiles * splits
  int stages;              // depth of the shared-memory ring
  int cmax;                // FUSED: most chunks an item has (resident B tiles)
  int dbg;                 // tuning build only
  // 1: the CTAs that share a tile (one per K split) form a thread-block cluster, every CTA has
  // exactly one item, and the partial sums travel through the shared memory of the cluster's first
  // CTA instead of global scratch and an atomic counter
  int cluster;
  // Grouped launches (the selected experts of a mixture-of-experts layer): the items are the 128-row
  // tiles of `gmats` matrices of each live work entry, every entry with its own weights, prepared
  // activations, tables and result rows; no K split.  batch is the instantiation's MB, out_dim the
  // pitch of a result row (gmats matrices of gtpe * 128 rows side by side).
  const MmaGroupEntry* gwork;
  const int* gcount;  // live entries (device memory, written by the kernel that routed the tokens)
  int gmax;           // entries the launch was sized for
  int gtpe;           // 128-row tiles per matrix
  int gmats;          // matrices per entry
  int gfirst;         // the first of them in MmaGroupEntry::w
  int gdirect;        // result row of activation m: 0 -> entry * MB + m, 1 -> the entry's item[m]
  int gtab;           // floats of tables per entry
  size_t gxb;         // bytes of prepared B operand per entry
};

// Shared-memory plan (dynamic, 1024-byte aligned base): ring of stages (weights then meta),
// 2 B tiles (8 K-steps x N rows x 32 bytes), per-(row,group) tables {sum x, 2^(E-26), 2^(26-E)},
// mbarriers, the TMEM base holder.
// FUSED: the activation digits are made by the kernel itself, for the K range of the CTA's items
// only (at most `cmax` chunks), and stay resident after the ring instead of travelling with every
// stage.
// C: chunks of 256 elements per stage.  The nibble formats take two: what a stage costs every role
// in waits, fences and arrivals is then paid once per 36 KiB instead of once per 18 KiB.  A stage's
// layout is [C weight blocks][C B tiles].
// Rows of 128 partial sums the first CTA of a cluster can receive: (splits - 1) x activation rows.
constexpr int kClusterRecvRows = 7;

template <int N, int FMT = FMT_MLX4, bool FUSED = false, int C = 1>
struct MmaSmem {
  static constexpr int kBTileBytes = 8 * N * 32;  // 256 K-bytes for each of N rows
  static constexpr int kStage = C * (Fmt<FMT>::kStageBytes + (FUSED ? 0 : kBTileBytes));
  static __host__ __device__ size_t bytes(int stages, int batch, int in_dim, int cmax = 0) {
    return (size_t)stages * kStage + (FUSED ? (size_t)cmax * kBTileBytes : 0) +
           (size_t)batch * (in_dim / Fmt<FMT>::kGroup) * 8 + 1024 + 512 + 8 * kTileRows * 4 + kClusterRecvRows * kTileRows * 4;
  }
};

// Walks the (tile, chunk) stages of this CTA's work items in the order every role uses.
// G (grouped launches): the CTA takes one contiguous range of the live items, so that it stays with
// one entry's activations for several tiles; item w = (entry, matrix, tile of the matrix).
template <bool G>
struct StageWalkT {
  int w, tile, split, c, c1;
  int cps;  // chunks per stage
  int wend, entry, mat;  // G only
  __device__ __forceinline__ void open(const MmaArgs& a) {
    if (G) {
      const int per = a.gtpe * a.gmats;
      entry = w / per;
      const int rem = w - entry * per;
      mat = rem / a.gtpe;
      tile = rem - mat * a.gtpe;
      split = 0;
      c = 0;
      c1 = a.nchunks;
    } else {
      tile = w / a.splits;
      split = w - tile * a.splits;
      c = split * a.nchunks / a.splits;
      c1 = (split + 1) * a.nchunks / a.splits;
    }
  }
  __device__ __forceinline__ StageWalkT(const MmaArgs& a, int chunks_per_stage = 1, int live_items = 0)
      : w(blockIdx.x), cps(chunks_per_stage) {
    if (G) {
      w = (int)((long long)blockIdx.x * live_items / gridDim.x);
      wend = (int)((long long)(blockIdx.x + 1) * live_items / gridDim.x);
    }
    if (live(a)) open(a);
  }
  __device__ __forceinline__ bool live(const MmaArgs& a) const { return G ? w < wend : w < a.items; }
  // chunks of the current stage (an item with an odd number of chunks ends on a stage of one)
  __device__ __forceinline__ int nc() const { return c1 - c < cps ? c1 - c : cps; }
  __device__ __forceinline__ bool last_chunk() const { return c + nc() == c1; }
  __device__ __forceinline__ void next(const MmaArgs& a) {
    c += nc();
    if (c == c1) {
      w += G ? 1 : gridDim.x;
      if (live(a)) open(a);
    }
  }
};

// ---- activation preparation -----------------------------------------------------------------
// One block of 64 threads per (activation row, 64-element group): group sum, power-of-two scale,
// and the base-128 digits of every element written where the tensor core expects them:
// chunk (256 K) -> K-step (32) -> half (16 bytes) -> 8-row core matrix -> row -> byte.
// G32: sums and scales per 32 elements (one warp each) instead of per 64.  NATURAL: the B bytes of
// a K step in element order (for A operands that lie in memory in element order) instead of the
// order the nibble converters produce.
template <int DIGITS, bool G32 = false, bool NATURAL = false, bool PAIRH = false>
__global__ void __launch_bounds__(64)
mlx_prep_x_kernel(const float* __restrict__ x, unsigned char* __restrict__ xb, float* __restrict__ xtab, int batch,
                  int in_dim, int N) {
  constexpr int QBITS = DIGITS == 4 ? 26 : 19;  // |q| <= 2^QBITS keeps the top digit within a signed byte
  constexpr bool PAIRED = G32 && !NATURAL;      // Q4_K: see Fmt::kPaired
  const int groups = in_dim / 64;
  const int m = blockIdx.x / groups, g = blockIdx.x - m * groups;
  const int t = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();  // x may be the output of the kernel in front
  const float v = x[(size_t)m * in_dim + g * 64 + t];
  float s = v, mx = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (!G32) {
    __shared__ float sh[4];
    if ((t & 31) == 0) {
      sh[t >> 5] = s;
      sh[2 + (t >> 5)] = mx;
    }
    __syncthreads();
    s = sh[0] + sh[1];
    mx = fmaxf(sh[2], sh[3]);
  }
  int e = (int)((__float_as_uint(mx) >> 23) & 0xFF);  // mx < 2^(e-126)
  if (e < QBITS + 2) e = QBITS + 2;
  if (e > 254) e = 254;  // inf/nan inputs: results are undefined, not a hang
  if (G32) {
    if ((t & 31) == 0) {
      const int g32 = 2 * g + (t >> 5), n32 = 2 * groups;
      xtab[m * n32 + g32] = s;
      xtab[(batch + m) * n32 + g32] = __uint_as_float((uint32_t)(e - 126 - QBITS + 127) << 23);
    }
  } else if (t == 0) {
    xtab[m * groups + g] = s;
    xtab[(batch + m) * groups + g] = __uint_as_float((uint32_t)(e - 126 - QBITS + 127) << 23);  // 2^(E-QBITS)
  }
  const float fi = __uint_as_float((uint32_t)(QBITS - (e - 126) + 127) << 23);
  int q = __float2int_rn(v * fi);
  // position of element k inside its chunk's B tile
  const int k = (g & 3) * 64 + t;          // element within the 256-element chunk
  const int step = k >> 5, w = (k & 31) >> 3, j = k & 7;
  const int pos = NATURAL ? (k & 31) : 8 * w + 4 * (j & 1) + (j >> 1);  // byte along K inside the step (order of the A bytes)
  const size_t base = (size_t)(g >> 2) * (N * 256) + step * (N * 32) + (pos >> 4) * ((N / 8) * 128) + (pos & 15);
  const int db = N / 2;
#pragma unroll
  for (int d = 0; d < DIGITS; ++d) {
    int dig = d == DIGITS - 1 ? q : ((q + 64) & 127) - 64;
    q = (q - dig) >> 7;
    int n = m * DIGITS + d;
    if (PAIRED || PAIRH) {  // the other scale group's half of the rows holds zeros at this K position
      const bool second = PAIRH ? (pos & 16) != 0 : (step & 1) != 0;  // Q6_K: by the half of the step; Q4_K: by the step
      const int other = n + (second ? 0 : db);
      n += second ? db : 0;
      xb[base + (other >> 3) * 128 + (other & 7) * 16] = 0;
    }
    xb[base + (n >> 3) * 128 + (n & 7) * 16] = (unsigned char)(dig & 0xFF);
  }
}

// The same preparation done by a CTA of the product kernel for itself (all warps, before the
// pipeline starts): digits into the resident B tiles in shared memory, sums and scales into the
// tables the epilogue reads.  A warp takes one 64-element group at a time, lane l the elements l
// and l + 32; the arithmetic and its order are those of mlx_prep_x_kernel.
template <int DIGITS, bool G32, bool NATURAL, int N, bool PAIRH = false>
__device__ __forceinline__ void prep_x_in_cta(const float* __restrict__ x, int batch, int in_dim, unsigned char* bres,
                                              float* xsum, float* xfs, int warp, int lane, int nwarps, int cbegin, int cend) {
  constexpr int QBITS = DIGITS == 4 ? 26 : 19;
  constexpr bool PAIRED = G32 && !NATURAL;
  constexpr int db = N / 2;
  const int groups = in_dim / 64;
  const int ntab = G32 ? 2 * groups : groups;
  const int gbegin = 4 * cbegin, gcount = 4 * (cend - cbegin);  // the 64-element groups of chunks [cbegin, cend)
  for (int gi = warp; gi < batch * gcount; gi += nwarps) {
    const int m = gi / gcount, g = gbegin + (gi - m * gcount);
    const float* xp = x + (size_t)m * in_dim + g * 64;
    float v[2] = {xp[lane], xp[32 + lane]};
    float s[2] = {v[0], v[1]}, mx[2] = {fabsf(v[0]), fabsf(v[1])};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        s[h] += __shfl_xor_sync(0xffffffffu, s[h], o);
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], o));
      }
    }
    if (!G32) {
      s[0] = s[1] = s[0] + s[1];
      mx[0] = mx[1] = fmaxf(mx[0], mx[1]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int e = (int)((__float_as_uint(mx[h]) >> 23) & 0xFF);
      if (e < QBITS + 2) e = QBITS + 2;
      if (e > 254) e = 254;
      if (lane == 0 && (G32 || h == 0)) {
        const int ti = m * ntab + (G32 ? 2 * g + h : g);
        xsum[ti] = s[h];
        xfs[ti] = __uint_as_float((uint32_t)(e - 126 - QBITS + 127) << 23);
      }
      const float fi = __uint_as_float((uint32_t)(QBITS - (e - 126) + 127) << 23);
      int q = __float2int_rn(v[h] * fi);
      const int k = (g & 3) * 64 + h * 32 + lane;  // element within the 256-element chunk
      const int step = k >> 5, w = (k & 31) >> 3, j = k & 7;
      const int pos = NATURAL ? (k & 31) : 8 * w + 4 * (j & 1) + (j >> 1);
      unsigned char* base = bres + (size_t)((g >> 2) - cbegin) * (N * 256) + step * (N * 32) + (pos >> 4) * ((N / 8) * 128) + (pos & 15);
#pragma unroll
      for (int d = 0; d < DIGITS; ++d) {
        int dig = d == DIGITS - 1 ? q : ((q + 64) & 127) - 64;
        q = (q - dig) >> 7;
        int n = m * DIGITS + d;
        if (PAIRED || PAIRH) {
          const bool second = PAIRH ? (pos & 16) != 0 : (step & 1) != 0;
          const int other = n + (second ? 0 : db);
          n += second ? db : 0;
          base[(other >> 3) * 128 + (other & 7) * 16] = 0;
        }
        base[(n >> 3) * 128 + (n & 7) * 16] = (unsigned char)(dig & 0xFF);
      }
    }
  }
}

// N: B rows (accumulator columns) per group block; DIGITS: base-128 digits per activation;
// MB: activation rows the instantiation can take (MB * DIGITS <= N).
template <int N, int DIGITS, int MB, int FMT = FMT_MLX4, bool FUSED = false, int C = 1, bool G = false>
__global__ void __launch_bounds__((mma_threads<N, FMT>()), 1)
mlx_mma_kernel(const __grid_constant__ MmaArgs a) {
  static_assert(!G || (!FUSED && FMT == FMT_MLX4), "grouped launches: MLX 4-bit, activations prepared in front");
  TP(const long long t_entry = clock64();)
  typedef StageWalkT<G> StageWalk;
  constexpr int EP = epi_parts<N, FMT>();
  constexpr int kEpiWarps = 4 * EP, kEpiThreads = kEpiWarps * 32;
  constexpr int kWarpTMA = kConvWarps + kEpiWarps, kWarpMMA = kWarpTMA + 1;
  constexpr int kThreads = mma_threads<N, FMT>();
  static_assert(MB * DIGITS * (Fmt<FMT>::kHalves ? 2 : 1) <= N, "the digits of the activation rows must fit the N columns");
  static_assert(N == 8 || N == 16 || N == 32, "accumulator blocks of 8, 16 or 32 columns");
  typedef Fmt<FMT> F;
  constexpr int kBlocks = F::kBlocks;
  constexpr int kACols = F::kConv ? 64 * C : 0;  // TMEM columns of one A buffer (a stage)
  constexpr int kDCols = C * kBlocks * N;        // accumulator columns of a stage
  // Depths of the A ring and of the accumulator ring in TMEM (512 columns).  A third A buffer lets
  // the converters start stage i+2 while the MMAs of stage i still run; where the columns do not
  // allow four of each, the accumulators, which the epilogue drains quickly, get the shallower ring.
  constexpr int NA = (kACols + kDCols) * 4 <= 512 ? 4 : (3 * kACols + 2 * kDCols <= 512 ? 3 : 2);
  constexpr int ND = (kACols + kDCols) * 4 <= 512 ? 4 : 2;
  static_assert(NA * kACols + ND * kDCols <= 512, "TMEM plan");
  static_assert(C == 1 || F::kConv, "two chunks per stage are for the formats that convert");
  constexpr uint32_t kCols = 512;
  constexpr int kStage = MmaSmem<N, FMT, FUSED, C>::kStage;
  constexpr int kStageBytes = F::kStageBytes, kStageWBytes = F::kStageWBytes;
  constexpr int kBTileBytes = MmaSmem<N, FMT, FUSED, C>::kBTileBytes;
  constexpr int kStageLoad = kStageBytes + (FUSED ? 0 : kBTileBytes);  // bytes a chunk brings into a stage
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  const int S = a.stages;
  unsigned char* ring = smem;
  const int groups = a.in_dim / F::kGroup;
  unsigned char* bres = ring + (size_t)S * kStage;  // FUSED: resident B tiles of every chunk
  float* xsum = reinterpret_cast<float*>(bres + (FUSED ? (size_t)a.cmax * kBTileBytes : 0));  // [batch][groups] sum of x
  float* xfs = xsum + (size_t)a.batch * groups;                        // [batch][groups] 2^(E-QBITS)
  uint64_t* bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(xfs + (size_t)a.batch * groups) + 15) & ~uintptr_t(15));
  // bars: full[S], empty[S], a_ready[NA], a_free[NA], d_full[ND], d_free[ND], cluster
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 2 * NA + 2 * ND + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* pair = reinterpret_cast<float*>(tmem_holder + 4);  // [EP-1][MB][128]: the sums of an item from the epilogue parts above 0
  static_assert((EP - 1) * MB <= 8, "room for the parts' sums");
  float* recv = pair + 8 * kTileRows;  // [splits-1][MB][128]: partial sums from the cluster's other CTAs (first CTA only)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + S);
  const uint32_t aready0 = smem_u32(bars + 2 * S), afree0 = aready0 + 8 * NA;
  const uint32_t mdone0 = afree0 + 8 * NA, dfree0 = mdone0 + 8 * ND;  // mdone: a stage's accumulators are complete
  const uint32_t clbar = dfree0 + 8 * ND;  // cluster launches: the other CTAs' partial sums have arrived (one arrival per warp)

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);
      // converters (conversion formats), epilogue (scale data), MMA commit (B tile, A read from the stage)
      // (one arrival per warp: a warp's lanes meet first and one of them arrives for all)
      mbar_init(empty0 + 8 * s, (F::kConv ? kConvWarps / 2 : 0) + kEpiWarps + 1);
    }
    for (int b = 0; b < NA; ++b) {
      mbar_init(aready0 + 8 * b, kConvWarps / 2);
      mbar_init(afree0 + 8 * b, 1);
    }
    for (int b = 0; b < ND; ++b) {
      mbar_init(mdone0 + 8 * b, 1);
      mbar_init(dfree0 + 8 * b, kEpiWarps);
    }
    if (a.cluster) mbar_init(clbar, 4 * (a.splits - 1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kWarpMMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_launch_dependents();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (a.cluster) cluster_sync_all();  // the first CTA's barrier is initialised before any peer can arrive on it
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmemA0 = tmem_base, tmemD0 = tmem_base + NA * kACols;  // A: NA x kACols; D: ND x kDCols
  bool ok = true;
  int gitems = 0;
  if (G) {
    pdl_wait();  // the work entries come from the kernels in front
    int n = __ldcg(a.gcount);
    if (n > a.gmax) n = a.gmax;
    gitems = n * a.gtpe * a.gmats;
  }
  StageWalk sw(a, C, gitems);
  // where a stage's weights and prepared activations lie
  auto wsrc = [&](const StageWalk& s) {
    const unsigned char* base = a.w;
    if (G) base = reinterpret_cast<const unsigned char*>(__ldg(reinterpret_cast<const unsigned long long*>(&a.gwork[s.entry].w[a.gfirst + s.mat])));
    return base + ((size_t)s.tile * a.nchunks + s.c) * kStageBytes;
  };
  auto bsrc = [&](const StageWalk& s) { return a.xb + (G ? (size_t)s.entry * a.gxb : 0) + (size_t)s.c * kBTileBytes; };
  TP(const bool tr = blockIdx.x == gridDim.x / 2 && (!(a.dbg & 8) || a.gmats == 2); if (tr && tid == 0) { g_mma_trace[7][0] = clock64(); g_mma_trace[7][3] = t_entry; })
  const int cbase = sw.live(a) ? sw.c : 0;  // first chunk of this CTA's K range

  if (FUSED) {
    // The weights do not depend on the kernel in front: the producer fills the ring, then every
    // warp helps to turn the activations into digits, sums and scales.
    if (warp == kWarpTMA && lane == 0) {
      StageWalk sw0 = sw;
      for (int i = 0; i < S && i < kFirstStages && sw0.live(a); ++i, sw0.next(a)) {
        mbar_expect_tx(full0 + 8 * i, sw0.nc() * kStageBytes);
        bulk_load_1d(smem_u32(ring + (size_t)i * kStage), wsrc(sw0), sw0.nc() * kStageBytes, full0 + 8 * i);
      }
    }
    pdl_wait();
    // every item of this CTA covers the same K range (the grid is a multiple of the K splits)
    if (sw.live(a))
      prep_x_in_cta<DIGITS, FMT != FMT_MLX4, !F::kConv, N, FMT == FMT_Q6K>(a.x, a.batch, a.in_dim, bres, xsum, xfs, warp, lane, kThreads / 32,
                                                                 sw.c, sw.c1);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the MMA reads the digits through the async proxy
    __syncthreads();
  }

  if (warp == kWarpTMA) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // The weights do not depend on the kernel in front: fill the ring with them first, then
      // wait for the activation digits and add the B tiles of those stages.
      int i = 0;
      if (FUSED) {
        for (; i < S && i < kFirstStages && sw.live(a); ++i) sw.next(a);  // asked for before the activations were prepared
      } else {
        StageWalk sw0 = sw;
        for (; i < S && i < kFirstStages && sw0.live(a); ++i, sw0.next(a)) {
          uint32_t dst = smem_u32(ring + (size_t)i * kStage);
          mbar_expect_tx(full0 + 8 * i, sw0.nc() * kStageLoad);
          bulk_load_1d(dst, wsrc(sw0), sw0.nc() * kStageBytes, full0 + 8 * i);
        }
        pdl_wait();
        for (int j = 0; j < i; ++j, sw.next(a))
          bulk_load_1d(smem_u32(ring + (size_t)j * kStage) + C * kStageBytes, bsrc(sw), sw.nc() * kBTileBytes, full0 + 8 * j);
      }
      for (; sw.live(a) && ok; ++i, sw.next(a)) {
        int slot = i % S, round = i / S;
        if (round > 0) ok = mbar_wait(empty0 + 8 * slot, (round - 1) & 1, a.status, 1);
        else if (i == kFirstStages) ok = mbar_wait(full0, 0, a.status, 11);  // the first stage is in: the rest of the ring may follow
        if (!ok) break;
        uint32_t dst = smem_u32(ring + (size_t)slot * kStage);
        mbar_expect_tx(full0 + 8 * slot, sw.nc() * kStageLoad);
        bulk_load_1d(dst, wsrc(sw), sw.nc() * kStageBytes, full0 + 8 * slot);
        if (!FUSED) bulk_load_1d(dst + C * kStageBytes, bsrc(sw), sw.nc() * kBTileBytes, full0 + 8 * slot);
        TP(if (tr && i < 64) g_mma_trace[0][i] = clock64();)
      }
    }
  } else if (warp >= kWarpMMA) {
    // ------------------------------------------------------------------ MMA issuers
    // The whole warp walks its stages and waits; one elected lane issues.  (What the instructions
    // need is the same in all lanes and can live in uniform registers, which roughly halves the
    // cycles an issue costs against a single diverged thread.)
    {
      // instruction descriptor: D s32, A u8 (nibbles) or s8 (Q8_0 bytes), B s8, both K-major, N, M=128
      const uint32_t idesc = (2u << 4) | (((FMT == FMT_Q80 || FMT == FMT_Q6K) ? 1u : 0u) << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
      // A from shared memory (Q8_0): K-adjacent core matrices 16 row groups apart, row groups 128 B apart
      const uint64_t adesc_hi = ((uint64_t)(2048u >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
      constexpr uint32_t kLBO = (N / 8) * 128, kSBO = 128;  // K-adjacent / N-adjacent core matrices
      const uint64_t desc_hi = ((uint64_t)(kLBO >> 4) << 16) | ((uint64_t)(kSBO >> 4) << 32) | (1ull << 46);
      // Every role sees every stage in order, so no barrier phase is ever skipped (a parity wait
      // can only tell the current phase from the one before it).
      for (int i = 0; sw.live(a) && ok; ++i) {
        const int ba = i % NA, b = i % ND, slot = i % S;
        ok = mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 8);
        if (ok && F::kConv) ok = mbar_wait(aready0 + 8 * ba, (i / NA) & 1, a.status, 2);
        if (ok && i >= ND) ok = mbar_wait(dfree0 + 8 * b, ((i - ND) / ND) & 1, a.status, 5);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        TP(if (tr && lane == 0 && i < 64) g_mma_trace[1][i] = clock64();)
        const int nc = sw.nc();
        if (elect_one()) {
#pragma unroll
        for (int cc = 0; cc < C; ++cc) {
          if (cc < nc) {
            const uint32_t bbase = FUSED ? smem_u32(bres + (size_t)(sw.c - cbase + cc) * kBTileBytes)
                                         : smem_u32(ring + (size_t)slot * kStage + C * kStageBytes + cc * kBTileBytes);
            const uint32_t dcol = tmemD0 + b * kDCols + cc * (kBlocks * N), acol = tmemA0 + ba * kACols + cc * 64;
#pragma unroll
            for (int step = 0; step < 8; ++step) {  // K = 32 per step
              const uint64_t bdesc = desc_hi | (uint64_t)(((bbase + step * (N * 32)) >> 4) & 0x3FFF);
              if (F::kConv) {  // two steps accumulate into the block of their 64 elements
                umma_i8_ts(dcol + (step >> 1) * N, acol + step * 8, bdesc, idesc, step & 1);
              } else {
                const uint32_t abase = smem_u32(ring + (size_t)slot * kStage) + step * 4096;
                umma_i8_ss(dcol + step * N, adesc_hi | (uint64_t)((abase >> 4) & 0x3FFF), bdesc, idesc, 0);
              }
            }
          }
        }
        umma_commit(mdone0 + 8 * b);
        if (F::kConv) umma_commit(afree0 + 8 * ba);
        umma_commit(empty0 + 8 * slot);
        }
        __syncwarp();
        TP(if (tr && lane == 0 && i < 64) g_mma_trace[2][i] = clock64();)
        sw.next(a);
      }
    }
  } else if (warp < kConvWarps && !F::kConv) {
    // nothing to convert: the MMA reads the stage as it lies
  } else if (warp < kConvWarps) {
    // ------------------------------------------------------------------ converters
    // Two groups of four warps convert alternate stages (thread = row r of the tile), so two stages
    // are in conversion at any time: a stage's conversion is a fixed latency of well over a
    // thousand cycles whatever its size, and what counts is how many run side by side.  Both groups
    // follow every stage's barriers in order, also those of the stages they do not convert, so no
    // barrier phase is ever skipped (a parity wait can only tell the current phase from the one
    // before it).
    const int q4 = warp & 3, grp = warp >> 2;
    const int r = q4 * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    for (int i = 0; sw.live(a) && ok; ++i, sw.next(a)) {
      const int ba = i % NA, slot = i % S;
      ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 4));
      if (ok && i >= NA) ok = __all_sync(0xffffffffu, mbar_wait(afree0 + 8 * ba, ((i - NA) / NA) & 1, a.status, 3));
      if (!ok) break;
      if ((i & 1) != grp) continue;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      TP(if (tr && q4 == 0 && lane == 0 && i < 64) g_mma_trace[3][i] = clock64();)
      const unsigned char* st = ring + (size_t)slot * kStage;
      // ---- this row of each chunk of the stage: 256 nibbles -> 256 bytes -> 64 TMEM columns ----
      const int nc = sw.nc();
#pragma unroll
      for (int cc = 0; cc < C; ++cc) {
        if (cc < nc) {
          uint4 qv[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (DBG(2)) qv[u] = make_uint4(r, u, cc, i);  // tuning: no shared-memory loads
            else qv[u] = *reinterpret_cast<const uint4*>(st + cc * kStageBytes + r * 128 + ((u ^ (r & 7)) << 4));
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            uint32_t ws[4] = {qv[u].x, qv[u].y, qv[u].z, qv[u].w};
            uint32_t regs[8];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              regs[2 * w + 0] = ws[w] & 0x0F0F0F0Fu;         // elements 0,2,4,6 of the word
              regs[2 * w + 1] = (ws[w] >> 4) & 0x0F0F0F0Fu;  // elements 1,3,5,7
            }
            if (!DBG(1)) tmem_st8(tmemA0 + lane_base + ba * kACols + cc * 64 + u * 8, regs);
            else if ((regs[0] ^ regs[3] ^ regs[5] ^ regs[7]) == 0x12345678u) *last_flag = 1;  // tuning: no TMEM stores
          }
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      // One arrival per warp: 128 arrivals on one mbarrier serialise in the shared-memory atomic
      // unit and cost more than the conversion itself.  The lanes meet (which also orders their
      // shared-memory reads and TMEM stores before the elected lane's releasing arrival).
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(aready0 + 8 * ba);
        mbar_arrive(empty0 + 8 * slot);
      }
      TP(if (tr && q4 == 0 && lane == 0 && i < 64) g_mma_trace[4][i] = clock64();)
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // EP warps per TMEM lane quarter: part p takes the p-th share of a stage's accumulator
    // blocks; each keeps its own running sums and the parts are added, in order, when an item
    // (tile, K range) ends.
    const int q4 = warp & 3, half = (warp - kConvWarps) >> 2;  // half: the part, 0 .. EP-1
    const int r = q4 * 32 + lane;  // row of the tile == TMEM lane
    const int et = tid - kConvThreads;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    float acc[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = 0.f;
    if (!FUSED && !G) {
      pdl_wait();  // the tables come from the preparation kernel in front
      for (int i = et; i < 2 * a.batch * groups; i += kEpiThreads) xsum[i] = __ldg(a.xtab + i);
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
    }
    int nb = a.batch;    // activation rows in use (G: of the current entry)
    int cur_entry = -1;  // G: the entry whose tables are in shared memory
    int orow[G ? MB : 1];  // G: result row of each activation row
    constexpr int kHB = kBlocks / EP;                       // blocks of this part
    constexpr int kSub = kHB * N <= 64 ? kHB : 64 / N;      // blocks per pass (at most 64 columns in registers)
    constexpr bool kNarrow = kSub * N == 8;                 // a pass of one 8-column block: one 8-column load
    constexpr int NLD = kNarrow ? 1 : kSub * N / 16;        // 16-column loads per pass
    for (int i = 0; sw.live(a) && ok; ++i) {
      int b = i % ND, slot = i % S;
      if (G && sw.entry != cur_entry) {
        // a new entry: its tables, row count and result rows.  Every epilogue thread passed the barrier
        // that ends the item before, so nobody still reads the old tables.
        cur_entry = sw.entry;
        const float* tab = a.xtab + (size_t)cur_entry * a.gtab;
        for (int j = et; j < 2 * a.batch * groups; j += kEpiThreads) xsum[j] = __ldcg(tab + j);
        const MmaGroupEntry* ge = a.gwork + cur_entry;
        nb = __ldg(&ge->count);
#pragma unroll
        for (int m = 0; m < (G ? MB : 1); ++m) orow[m] = a.gdirect ? __ldg(&ge->item[m]) : cur_entry * MB + m;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      }
      ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 6));
      uint4 mvs[C];
      uint32_t q6d = 0;  // Q6_K: the super-block's f16 d (the 16 int8 scales are in mvs)
      const int nc = sw.nc();
      if (ok) {
        uint32_t seen = 1u;
#pragma unroll
        for (int cc = 0; cc < C; ++cc) {
          mvs[cc] = make_uint4(0, 0, 0, 0);
          const unsigned char* mrow = ring + (size_t)slot * kStage + cc * kStageBytes + kStageWBytes + r * F::kMetaRow;
          if (cc < nc) mvs[cc] = *reinterpret_cast<const uint4*>(mrow);
          if (FMT == FMT_Q6K) q6d = *reinterpret_cast<const uint32_t*>(mrow + 16);
          seen |= mvs[cc].x | q6d;
        }
        // the scale data is in registers: one lane releases the stage for the warp (the values are
        // consumed by the shuffle, so every lane's loads have completed before the arrival)
        seen = __reduce_or_sync(0xffffffffu, seen);
        if (lane == 0 && seen) mbar_arrive(empty0 + 8 * slot);
        ok = __all_sync(0xffffffffu, mbar_wait(mdone0 + 8 * b, (i / ND) & 1, a.status, 7));
      }
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      TP(if (tr && et == 0 && i < 64) g_mma_trace[5][i] = clock64();)
#pragma unroll
      for (int cc = 0; cc < C; ++cc) {
      if (cc < nc) {
      const uint32_t meta[4] = {mvs[cc].x, mvs[cc].y, mvs[cc].z, mvs[cc].w};
      const int gbase = (sw.c + cc) * kBlocks;
#pragma unroll
      for (int sub = 0; sub < kHB / kSub; ++sub) {
        const int blk0 = half * kHB + sub * kSub;  // first block of this pass
        uint32_t t[NLD][16];
#pragma unroll
        for (int l = 0; l < NLD; ++l) {
          const uint32_t taddr = tmemD0 + lane_base + b * kDCols + cc * (kBlocks * N) + blk0 * N + l * 16;
          if (kNarrow) tmem_ld8(taddr, *reinterpret_cast<uint32_t(*)[8]>(&t[l][0]));
          else tmem_ld16(taddr, t[l]);
        }
#pragma unroll
        for (int l = 0; l < NLD; ++l) {
          if (kNarrow) tmem_wait_ld(*reinterpret_cast<uint32_t(*)[8]>(&t[l][0]));
          else tmem_wait_ld(t[l]);
        }
        TP(if (tr && et == 0 && i == 2) g_mma_trace[7][12 + 2 * cc] = clock64();)
        if (sub == kHB / kSub - 1 && cc == nc - 1) {  // the stage's last load: its accumulators are free
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(dfree0 + 8 * b);
        }
#pragma unroll
        for (int g = 0; g < kSub; ++g) {
          const int blk = blk0 + g;
          auto col = [&](int cidx) { return (int)t[(g * N + cidx) >> 4][(g * N + cidx) & 15]; };
          auto digits_dot = [&](int c0) {  // the integer dot of the DIGITS columns from c0
            if (DIGITS == 4) {
              int lo = col(c0) + (col(c0 + 1) << 7), hi = col(c0 + 2) + (col(c0 + 3) << 7);
              return fmaf((float)hi, 16384.f, (float)lo);
            }
            int lo = col(c0) + (col(c0 + 1) << 7);
            return fmaf((float)col(c0 + 2), 16384.f, (float)lo);
          };
          if (FMT == FMT_Q4K) {
            // the block holds two 32-element sub-blocks: columns [0, N/2) and [N/2, N); their
            // multipliers (sc*d) and -(m*dmin), each rounded to f32 as dequantRowQ4KTo does
            constexpr int db = N / 2;
            const float d16 = __half2float(__ushort_as_half((unsigned short)(meta[0] & 0xFFFFu)));
            const float dmin16 = __half2float(__ushort_as_half((unsigned short)(meta[0] >> 16)));
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int sub = 2 * blk + hh, bit = 12 * sub, wi = bit >> 5, sh = bit & 31;
              const uint32_t lo = wi == 0 ? meta[1] : wi == 1 ? meta[2] : meta[3];
              const uint32_t hi = wi == 0 ? meta[2] : wi == 1 ? meta[3] : 0u;
              const uint32_t f = __funnelshift_r(lo, hi, sh) & 0xFFFu;
              // Integer -> float through the exponent trick (an add and a subtract on the full-rate
              // pipes; eight sub-blocks a chunk would otherwise queue on the conversion unit).  Exact
              // while |v| < 2^22: the 6-bit fields trivially, and a column sums 32 products of a
              // nibble and a digit in [-64, 63], so |c0 + 128 c1| <= 30720 * 129 < 2^22.
              auto small_f = [](uint32_t v) { return __uint_as_float(0x4B000000u | v) - 8388608.f; };
              auto int_f = [](int v) { return __int_as_float(0x4B400000 + v) - 12582912.f; };
              const float sc = __fmul_rn(small_f(f & 63u), d16), bi = -__fmul_rn(small_f(f >> 6), dmin16);
              const int ti = 2 * gbase + sub;  // the sub-block's entry of the per-32 tables
              auto paired_dot = [&](int c0) {
                const float lo = int_f(col(c0) + (col(c0 + 1) << 7));
                const float hi = DIGITS == 4 ? int_f(col(c0 + 2) + (col(c0 + 3) << 7)) : int_f(col(c0 + 2));
                return fmaf(hi, 16384.f, lo);
              };
#pragma unroll
              for (int m = 0; m < MB; ++m) {
                if (MB == 1 || m < nb) {
                  const float dot = paired_dot(hh * db + DIGITS * m) * xfs[m * groups + ti];
                  acc[m] = fmaf(sc, dot, acc[m]);
                  acc[m] = fmaf(bi, xsum[m * groups + ti], acc[m]);
                }
              }
            }
          } else if (FMT == FMT_Q5K) {
            // one 32-element sub-block: (sc*d) and -(m*dmin), each rounded to f32 as dequantRowQ5K does
            const float d16 = __half2float(__ushort_as_half((unsigned short)(meta[0] & 0xFFFFu)));
            const float dmin16 = __half2float(__ushort_as_half((unsigned short)(meta[0] >> 16)));
            const int bit = 12 * blk, wi = bit >> 5, sh = bit & 31;
            const uint32_t lo = wi == 0 ? meta[1] : wi == 1 ? meta[2] : meta[3];
            const uint32_t hi = wi == 0 ? meta[2] : wi == 1 ? meta[3] : 0u;
            const uint32_t f = __funnelshift_r(lo, hi, sh) & 0xFFFu;
            const float sc = __fmul_rn((float)(f & 63u), d16), bi = -__fmul_rn((float)(f >> 6), dmin16);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
              if (MB == 1 || m < nb) {
                const float dot = digits_dot(DIGITS * m) * xfs[m * groups + gbase + blk];
                acc[m] = fmaf(sc, dot, acc[m]);
                acc[m] = fmaf(bi, xsum[m * groups + gbase + blk], acc[m]);
              }
            }
          } else if (FMT == FMT_Q6K) {
            // the step's two 16-element scale groups: columns [0, N/2) and [N/2, N); multiplier
            // d * sc rounded to f32 as dequantRowQ6K does
            const float d16 = __half2float(__ushort_as_half((unsigned short)(q6d & 0xFFFFu)));
            const uint32_t sw4 = (blk >> 1) == 0 ? meta[0] : (blk >> 1) == 1 ? meta[1] : (blk >> 1) == 2 ? meta[2] : meta[3];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int s8 = (int)(signed char)((sw4 >> (8 * (2 * (blk & 1) + hh))) & 0xFFu);
              const float sc = __fmul_rn(d16, (float)s8);
#pragma unroll
              for (int m = 0; m < MB; ++m) {
                if (MB == 1 || m < nb) {
                  const float dot = digits_dot(hh * (N / 2) + DIGITS * m) * xfs[m * groups + gbase + blk];
                  acc[m] = fmaf(sc, dot, acc[m]);
                }
              }
            }
          } else {
            // the block's multiplier of the integer dot and of the block's sum of x
            float sc, bi;
            if (FMT == FMT_MLX4) {  // {scale, bias} bf16 pair of the 64-element group
              const uint32_t mw = blk == 0 ? meta[0] : blk == 1 ? meta[1] : blk == 2 ? meta[2] : meta[3];
              sc = __uint_as_float(mw << 16);
              bi = __uint_as_float(mw & 0xFFFF0000u);
            } else {  // f16 block scale
              const uint32_t mw = (blk >> 1) == 0 ? meta[0] : (blk >> 1) == 1 ? meta[1] : (blk >> 1) == 2 ? meta[2] : meta[3];
              sc = __half2float(__ushort_as_half((unsigned short)((mw >> (16 * (blk & 1))) & 0xFFFFu)));
              bi = 0.f;
            }
#pragma unroll
            for (int m = 0; m < MB; ++m) {
              if (MB == 1 || m < nb) {
                const float dot = digits_dot(DIGITS * m) * xfs[m * groups + gbase + blk];
                acc[m] = fmaf(sc, dot, acc[m]);
                if (FMT != FMT_Q80) acc[m] = fmaf(bi, xsum[m * groups + gbase + blk], acc[m]);
              }
            }
          }
        }
      }
      TP(if (tr && et == 0 && i == 2) g_mma_trace[7][13 + 2 * cc] = clock64() + (long long)(__float_as_int(acc[0]) & 1);)
      }  // cc < nc
      }  // chunks of the stage
      TP(if (tr && et == 0 && i < 64) g_mma_trace[6][i] = clock64();)
      const bool item_done = sw.last_chunk();
      const int tile = sw.tile, split = sw.split;
      const int gmat = G ? sw.mat : 0;
      sw.next(a);
      if (!item_done) continue;
      // ---- the item is complete: add the parts' sums (parts above 0 -> shared memory -> part 0) ----
      if (half != 0) {
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          pair[((half - 1) * MB + m) * kTileRows + r] = acc[m];
          acc[m] = 0.f;
        }
      }
      TP(if (tr && et == 0 && i < 16) g_mma_trace[7][8] = clock64();)
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      TP(if (tr && et == 0 && i < 16) g_mma_trace[7][9] = clock64();)
      if (half == 0) {
#pragma unroll
        for (int m = 0; m < MB; ++m) {
#pragma unroll
          for (int p = 0; p < EP - 1; ++p) acc[m] += pair[(p * MB + m) * kTileRows + r];
        }
      }
      const int row = tile * kTileRows + r;
      if (a.cluster) {
        // The K splits of this tile are the CTAs of this cluster (rank == split) and each has this one
        // item.  Ranks above 0 put their sums into rank 0's shared memory and arrive on its barrier
        // (one releasing arrival per warp, after the warp's lanes have met); rank 0 waits, adds the
        // sums in split order — the same order as the scratch path, so the same bits — and stores.
        if (half == 0) {
          if (split != 0) {
#pragma unroll
            for (int m = 0; m < MB; ++m)
              if (m < a.batch) cluster_store_f32(cluster_map(smem_u32(recv + ((split - 1) * MB + m) * kTileRows + r), 0), acc[m]);
            __syncwarp();
            if (lane == 0) cluster_arrive_release(cluster_map(clbar, 0));
          } else {
            ok = __all_sync(0xffffffffu, mbar_wait_cluster(clbar, 0, a.status, 12));
            if (ok) {
#pragma unroll
              for (int m = 0; m < MB; ++m) {
                float sum = acc[m];
                for (int s2 = 1; s2 < a.splits; ++s2) sum += recv[((s2 - 1) * MB + m) * kTileRows + r];
                if (m < a.batch && row < a.out_dim) a.out[(size_t)m * a.out_dim + row] = sum;
              }
            }
          }
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m] = 0.f;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      } else if (G) {
        if (half == 0) {
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            if (m < nb) a.out[(size_t)orow[G ? m : 0] * a.out_dim + gmat * (a.gtpe * kTileRows) + row] = acc[m];
            acc[m] = 0.f;
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");  // pair and the tables are free for the next item
      } else if (a.splits == 1) {
        if (half == 0) {
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            if (m < a.batch && row < a.out_dim) a.out[(size_t)m * a.out_dim + row] = acc[m];
            acc[m] = 0.f;
          }
        }
        TP(if (tr && et == 0 && i < 16) g_mma_trace[7][10] = clock64();)
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");  // pair is free for the next item
        TP(if (tr && et == 0 && i < 16) g_mma_trace[7][11] = clock64();)
      } else {
        // Partial sums of this K range go to scratch; the CTA that arrives last at the tile adds the
        // partials in split order (so the result does not depend on arrival order) and stores.
        if (half == 0) {
          float* part = a.scratch + ((size_t)tile * a.splits + split) * (MB * kTileRows);
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            part[m * kTileRows + r] = acc[m];
            acc[m] = 0.f;
          }
          __threadfence();
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (et == 0) *last_flag = (atomicAdd(a.counters + tile, 1u) == (unsigned)a.splits - 1) ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (*last_flag && half == 0) {
          __threadfence();
          const float* base = a.scratch + (size_t)tile * a.splits * (MB * kTileRows);
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            float sum = 0.f;
            for (int s2 = 0; s2 < a.splits; ++s2) sum += __ldcg(base + (size_t)s2 * (MB * kTileRows) + m * kTileRows + r);
            if (m < a.batch && row < a.out_dim) a.out[(size_t)m * a.out_dim + row] = sum;
          }
          if (et == 0) a.counters[tile] = 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      }
    }
  }

  TP(if (tr && tid == 0) g_mma_trace[7][1] = clock64();)
  // ---- wind down: everyone meets, outstanding copies are drained, TMEM is returned ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
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
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kCols) : "memory");
  }
}

// ---- host side --------------------------------------------------------------------------

// Row-major words + {scale,bias} table -> tiled blocks; one thread per 16-byte unit / meta row.
__global__ void mlx_tile_kernel(const uint32_t* __restrict__ qw, const uint32_t* __restrict__ sb,
                                unsigned char* __restrict__ tiled, int out_dim, int in_dim, int ntiles, int nchunks) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t nblocks = (size_t)ntiles * nchunks;
  if (idx >= nblocks * (128 * 9)) return;
  size_t blk = idx / (128 * 9);
  int rem = (int)(idx - blk * (128 * 9));
  int tile = (int)(blk / nchunks), chunk = (int)(blk - (size_t)tile * nchunks);
  int r = rem / 9, u = rem - r * 9;
  int row = tile * 128 + r;
  uint4 v = make_uint4(0, 0, 0, 0);
  unsigned char* dst = tiled + blk * kStageBytes;
  if (u < 8) {
    if (row < out_dim) v = *reinterpret_cast<const uint4*>(qw + (size_t)row * (in_dim / 8) + chunk * 32 + u * 4);
    *reinterpret_cast<uint4*>(dst + r * 128 + ((u ^ (r & 7)) << 4)) = v;
  } else {
    if (row < out_dim) v = *reinterpret_cast<const uint4*>(sb + (size_t)row * (in_dim / 64) + chunk * 4);
    *reinterpret_cast<uint4*>(dst + kStageWBytes + r * 16) = v;
  }
}

bool mlx_mma_supported(const goph_mlx_weight* w) {
  return w->sb_bf16 && w->group_size == 64 && w->in_dim % kChunkK == 0 && w->in_dim <= 65536;
}

int mlx_mma_make_tiled(goph_mlx_weight* w) {
  int ntiles = (w->out_dim + kTileRows - 1) / kTileRows, nchunks = w->in_dim / kChunkK;
  size_t bytes = (size_t)ntiles * nchunks * kStageBytes;
  unsigned char* t = nullptr;
  GOPH_CUDA(cudaMalloc(&t, bytes));
  size_t threads = (size_t)ntiles * nchunks * 128 * 9;
  mlx_tile_kernel<<<(unsigned)((threads + 255) / 256), 256>>>(w->qweight, reinterpret_cast<const uint32_t*>(w->sb), t,
                                                              w->out_dim, w->in_dim, ntiles, nchunks);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(t);
    return fail_cuda(e, "mlx_tile_kernel");
  }
  w->tiled = t;
  w->bytes = bytes;
  return GOPH_OK;
}

struct MmaDeviceBufs {
  unsigned char* xb = nullptr;  // prepared B operand of the launch in flight
  float* xtab = nullptr;        // prepared per-(row, group) tables
  int* status = nullptr;
  float* scratch = nullptr;
  unsigned int* counters = nullptr;
};
// Fixed-size device scratch of the split-K fix-up: at most 2 x 160 items of 128 rows x 8
// activation rows, plus one counter per tile.  Allocated once per device.
constexpr size_t kScratchFloats = (size_t)2 * 160 * kTileRows * 8;
constexpr size_t kMaxCounters = 4096;
// Prepared activations: up to 8 rows of up to 65536 elements (B operand: 32 rows x in_dim bytes).
constexpr int kMaxPrepIn = 65536;  // mlx_mma_supported's bound on in_dim
constexpr size_t kPrepXbBytes = (size_t)32 * kMaxPrepIn;
constexpr size_t kPrepTabFloats = (size_t)2 * 8 * (kMaxPrepIn / 32);

// The buffers of a device are allocated on first use.  Nothing is published until every
// allocation has succeeded (a failure frees what it got and the next call tries again), and
// first calls from several threads are serialised.
static MmaDeviceBufs* device_bufs(int device) {
  static MmaDeviceBufs bufs[kMaxDevices];
  static bool ready[kMaxDevices] = {};
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (ready[device]) return &bufs[device];
  MmaDeviceBufs b;
  bool ok = cudaMalloc(&b.status, sizeof(int)) == cudaSuccess &&
            cudaMalloc(&b.scratch, kScratchFloats * sizeof(float)) == cudaSuccess &&
            cudaMalloc(&b.counters, kMaxCounters * sizeof(unsigned int)) == cudaSuccess &&
            cudaMalloc(&b.xb, kPrepXbBytes) == cudaSuccess &&
            cudaMalloc(&b.xtab, kPrepTabFloats * sizeof(float)) == cudaSuccess;
  ok = ok && cudaMemset(b.xb, 0, kPrepXbBytes) == cudaSuccess && cudaMemset(b.status, 0, sizeof(int)) == cudaSuccess &&
       cudaMemset(b.counters, 0, kMaxCounters * sizeof(unsigned int)) == cudaSuccess &&
       cudaDeviceSynchronize() == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    cudaFree(b.status);
    cudaFree(b.scratch);
    cudaFree(b.counters);
    cudaFree(b.xb);
    cudaFree(b.xtab);
    return nullptr;
  }
  bufs[device] = b;
  ready[device] = true;
  return &bufs[device];
}

void mlx_mma_status_clear(int device) {
  MmaDeviceBufs* b = device_bufs(device);
  if (b) cudaMemset(b->status, 0, sizeof(int));
}

int mlx_mma_status(int device) {
  MmaDeviceBufs* b = device_bufs(device);
  int v = -1;
  if (b) cudaMemcpy(&v, b->status, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

// A matrix in one of the tiled layouts, as the launch code sees it.
struct TiledDesc {
  const unsigned char* tiled;
  int device, out_dim, in_dim;
};

constexpr size_t kMmaSmemBudget = 222 * 1024;  // of the 227 KiB a CTA may have
constexpr int kMaxStages = 10;

// Clusters of `size` CTAs of the tensor-core GEMV that the device can hold at once (every such CTA
// takes a whole SM, so this is a property of how the SMs are grouped); asked once per device.
static int cluster_room(int device, int size);

// K split: enough (tile, split) items to occupy the SMs, bounded by the chunks and the scratch.
template <int MB>
static int choose_splits(const MmaArgs& a, int sm_count, int device) {
  int splits = 1;
  if (a.ntiles < sm_count) {
    splits = sm_count / a.ntiles;
    if (splits > a.nchunks) splits = a.nchunks;
    if (splits < 1) splits = 1;
    // The cheap way to add the splits' partial sums needs all clusters of `splits` CTAs resident at
    // once.  Where that many do not fit (48 tiles x 3: room for 45), fewer splits that do fit are the
    // better trade (6144 x 4096: 7.7 us with 2 splits in clusters against 8.3 us with 3 through scratch).
    if (options().mlx_cluster && splits > 2 && splits <= 8 && cluster_room(device, splits) < a.ntiles) {
      for (int s2 = splits - 1; s2 >= 2; --s2) {
        if (cluster_room(device, s2) >= a.ntiles) {
          splits = s2;
          break;
        }
      }
    }
  }
  if (options().mlx_splits > 0) splits = options().mlx_splits < a.nchunks ? options().mlx_splits : a.nchunks;
  while (splits > 1 && ((size_t)a.ntiles * splits * kTileRows * MB > kScratchFloats || (size_t)a.ntiles > kMaxCounters)) --splits;
  return splits;
}

int g_mma_dbg = 0;  // tuning build only

static int cluster_room(int device, int size) {
  static std::mutex mu;
  static int room[kMaxDevices][9];
  static bool known[kMaxDevices] = {};
  if (device < 0 || device >= kMaxDevices || size < 2 || size > 8) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (!known[device]) {
    auto kern = mlx_mma_kernel<8, 4, 1, FMT_MLX4, false, 2>;
    const size_t smem = 200 * 1024;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    for (int sz = 2; sz <= 8; ++sz) {
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = sz;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cudaLaunchConfig_t cfg;
      memset(&cfg, 0, sizeof cfg);
      cfg.gridDim = dim3(sz * 64);
      cfg.blockDim = dim3(mma_threads<8, FMT_MLX4>());
      cfg.dynamicSmemBytes = smem;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      room[device][sz] = n;
    }
    known[device] = true;
  }
  return room[device][size];
}

template <int N, int DIGITS, int MB, int FMT, bool FUSED, int C>
static int launch_impl(const TiledDesc& w, const MmaArgs& a0, cudaStream_t stream, bool prep, int stages, int splits) {
  MmaArgs a = a0;
  a.dbg = g_mma_dbg;
  DeviceState& st = device_state(w.device);
  a.stages = stages;
  a.splits = splits;
  a.items = a.ntiles * splits;
  a.cmax = (a.nchunks + splits - 1) / splits;
  size_t smem = MmaSmem<N, FMT, FUSED, C>::bytes(stages, a.batch, a.in_dim, a.cmax);
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!FUSED && prep) {
    // activations -> digits, sums and scales, once per launch
    cfg.gridDim = dim3(a.batch * (a.in_dim / 64));
    cfg.blockDim = dim3(64);
    note_launch();
    GOPH_CUDA(cudaLaunchKernelEx(&cfg, mlx_prep_x_kernel<DIGITS, FMT != FMT_MLX4, !Fmt<FMT>::kConv, FMT == FMT_Q6K>, a.x,
                                 const_cast<unsigned char*>(a.xb), const_cast<float*>(a.xtab), a.batch, a.in_dim, N));
  }
  auto kern = mlx_mma_kernel<N, DIGITS, MB, FMT, FUSED, C>;
  GOPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = a.items < st.sm_count ? a.items : st.sm_count;
  // FUSED: a CTA prepares the activations of one K range, so all its items must be of one split:
  // item w is split w % splits, and a grid that is a multiple of the splits keeps that fixed per CTA
  if (FUSED && a.items > grid) grid -= grid % splits;
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(mma_threads<N, FMT>());
  cfg.dynamicSmemBytes = smem;
  int cluster_room = -1;
  // K splits whose CTAs all run at once, one item each: the CTAs of a tile form a cluster and add
  // their partial sums through the first CTA's shared memory (no scratch, fence or atomic).  Only
  // when the device can hold every cluster of the grid at the same time — a second wave of clusters
  // would cost far more than the fix-up saves.
  if (options().mlx_cluster && splits > 1 && splits <= 8 && a.items == grid && (splits - 1) * MB <= kClusterRecvRows) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, size_t, int>, int> fits;  // (kernel, splits, smem, device) -> clusters resident at once
    const auto key = std::make_tuple((const void*)kern, splits, smem, w.device);
    int resident = -1;
    {
      std::lock_guard<std::mutex> lock(mu);
      auto it = fits.find(key);
      if (it != fits.end()) resident = it->second;
    }
    if (resident < 0) {
      if (cudaOccupancyMaxActiveClusters(&resident, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        resident = 0;
      }
      std::lock_guard<std::mutex> lock(mu);
      fits[key] = resident;
    }
    if (resident * splits >= grid) a.cluster = 1;
    else cfg.numAttrs = 1;
    cluster_room = resident;
  }
  // GOPH_TRACE_LAUNCH=1 in the environment: one line per tensor-core product with its launch plan
  static const bool trace = getenv("GOPH_TRACE_LAUNCH") != nullptr;
  if (trace)
    fprintf(stderr, "goph: mlx_mma_kernel fmt=%d out=%d in=%d rows=%d grid=%d splits=%d stages=%d chunks/stage=%d fused=%d cluster=%d (room for %d clusters)\n",
            FMT, a.out_dim, a.in_dim, a.batch, grid, splits, stages, C, (int)FUSED, a.cluster, cluster_room);
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  return GOPH_OK;
}

// Chunks per stage: two for the formats that convert, when a stage's A buffer and accumulators fit
// the tensor memory twice.
template <int N, int FMT>
constexpr int stage_chunks() {
  return (Fmt<FMT>::kConv && 2 * (2 * 64 + 2 * Fmt<FMT>::kBlocks * N) <= 512) ? 2 : 1;
}

template <int N, int DIGITS, int MB, int FMT, int C>
static int launch_with_chunks(const TiledDesc& w, const MmaArgs& a, cudaStream_t stream, bool prep) {
  const int sms = device_state(w.device).sm_count;
  const int splits = choose_splits<MB>(a, sms, w.device);
  const int cmax = (a.nchunks + splits - 1) / splits;
  // Narrow launches (one or two activation rows) whose items are short (at most four chunks: the
  // matrices that are split over K to fill the SMs) make the digits of their own K range inside
  // the product kernel: one launch instead of two (measured 7.3 against 7.6 us for 4096 x 4096 in
  // a dependent chain).  Longer items are served better by the separate kernel, whose small
  // blocks prepare the vector once for all CTAs (14336 x 4096: 14.1 against 15.2 us).
  // Option mlx_fuse = 0 always keeps the separate preparation kernel.
  if (N == 8 && options().mlx_fuse && splits <= sms && cmax <= 4) {
    size_t fixed = MmaSmem<N, FMT, true, C>::bytes(0, a.batch, a.in_dim, cmax);
    int stages = fixed < kMmaSmemBudget ? (int)((kMmaSmemBudget - fixed) / MmaSmem<N, FMT, true, C>::kStage) : 0;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages >= 3) return launch_impl<N, DIGITS, MB, FMT, N == 8, C>(w, a, stream, prep, stages, splits);
  }
  size_t fixed = MmaSmem<N, FMT, false, C>::bytes(0, a.batch, a.in_dim);
  int stages = fixed < kMmaSmemBudget ? (int)((kMmaSmemBudget - fixed) / MmaSmem<N, FMT, false, C>::kStage) : 0;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 3) {
    if (C > 1) return launch_with_chunks<N, DIGITS, MB, FMT, 1>(w, a, stream, prep);
    return fail(GOPH_E_UNSUPPORTED, "tensor-core path: activations of %d x %d leave no room for the ring", a.batch, a.in_dim);
  }
  return launch_impl<N, DIGITS, MB, FMT, false, C>(w, a, stream, prep, stages, splits);
}

template <int N, int DIGITS, int MB, int FMT>
static int launch_one(const TiledDesc& w, const MmaArgs& a, cudaStream_t stream, bool prep) {
  constexpr int C = stage_chunks<N, FMT>();
  if (C > 1 && options().mlx_chunks != 1) return launch_with_chunks<N, DIGITS, MB, FMT, C>(w, a, stream, prep);
  return launch_with_chunks<N, DIGITS, MB, FMT, 1>(w, a, stream, prep);
}

template <int FMT>
static int tiled_launch(const TiledDesc& w, float* out, const float* x, int batch, int digits, cudaStream_t stream,
                        bool x_prepared) {
  MmaDeviceBufs* bufs = device_bufs(w.device);
  if (!bufs) return fail(GOPH_E_NOMEM, "cannot allocate the tensor-core path's device scratch");
  MmaArgs a;
  memset(&a, 0, sizeof a);
  a.w = w.tiled;
  a.status = bufs->status;
  a.scratch = bufs->scratch;
  a.counters = bufs->counters;
  a.xb = bufs->xb;
  a.xtab = bufs->xtab;
  a.out_dim = w.out_dim;
  a.in_dim = w.in_dim;
  a.ntiles = (w.out_dim + kTileRows - 1) / kTileRows;
  a.nchunks = w.in_dim / kChunkK;
  // activation rows one launch can take: the accumulator blocks of a stage must fit TMEM twice
  constexpr bool kQ4K = Fmt<FMT>::kHalves;  // Q4_K and Q6_K need two columns per digit
  const int cap = kQ4K ? (digits == 3 ? 5 : 4) : 8;
  for (int b0 = 0; b0 < batch;) {
    int nb = batch - b0 < cap ? batch - b0 : cap;
    a.x = x + (size_t)b0 * w.in_dim;
    a.out = out + (size_t)b0 * w.out_dim;
    a.batch = nb;
    const bool prep = !(x_prepared && batch <= cap);
    int rc;
    if (digits == 3) {
      if (kQ4K && nb == 1) rc = launch_one<8, 3, 1, FMT>(w, a, stream, prep);
      else if (nb <= 2) rc = launch_one<kQ4K ? 16 : 8, 3, 2, FMT>(w, a, stream, prep);
      else if (nb <= 5) rc = launch_one<kQ4K ? 32 : 16, 3, 5, FMT>(w, a, stream, prep);
      else if (!kQ4K) rc = launch_one<32, 3, 8, kQ4K ? FMT_MLX4 : FMT>(w, a, stream, prep);
      else rc = fail(GOPH_E_UNSUPPORTED, "batch slice too wide");
    } else {
      if (nb == 1) rc = launch_one<8, 4, 1, FMT>(w, a, stream, prep);
      else if (nb == 2) rc = launch_one<kQ4K ? 16 : 8, 4, 2, FMT>(w, a, stream, prep);
      else if (nb <= 4) rc = launch_one<kQ4K ? 32 : 16, 4, 4, FMT>(w, a, stream, prep);
      else if (!kQ4K) rc = launch_one<32, 4, 8, kQ4K ? FMT_MLX4 : FMT>(w, a, stream, prep);
      else rc = fail(GOPH_E_UNSUPPORTED, "batch slice too wide");
    }
    if (rc) return rc;
    b0 += nb;
  }
  return GOPH_OK;
}

int mlx_mma_launch(const goph_mlx_weight* w, float* out, const float* x, int batch, int digits, cudaStream_t stream,
                   bool x_prepared) {
  if (!w->tiled) return fail(GOPH_E_UNSUPPORTED, "weight is not in the tiled layout");
  TiledDesc d{w->tiled, w->device, w->out_dim, w->in_dim};
  return tiled_launch<FMT_MLX4>(d, out, x, batch, digits, stream, x_prepared);
}

// ---- grouped launches (mixture-of-experts) -----------------------------------------------------

// The activations of every (entry, row) as the tensor core wants them: block = one row of one entry,
// a warp takes 64-element groups; arithmetic and layout are mlx_prep_x_kernel's.  PHASE 0: the row is
// the item's token in src[tokens][in_dim]; PHASE 1: silu(g) * u of the gate and up results
// src[entry * MB + m][2][in_dim] (kernels.SiLU then the multiply, backends/simd/kernels/activation.go:15-24;
// single-precision exp as in the CUDA-core expert kernels).
template <int N, int MB, int PHASE>
__global__ void __launch_bounds__(256)
moe_mma_prep_kernel(const MmaGroupEntry* __restrict__ work, const int* __restrict__ count, int max_entries,
                    const float* __restrict__ src, int in_dim, int top_k, unsigned char* __restrict__ xb, size_t xb_stride,
                    float* __restrict__ xtab, int tab_stride) {
  constexpr int DIGITS = 4, QBITS = 26;
  pdl_launch_dependents();
  pdl_wait();
  const int entry = blockIdx.x / MB, m = blockIdx.x - entry * MB;
  int live = __ldcg(count);
  if (live > max_entries) live = max_entries;
  if (entry >= live) return;
  const MmaGroupEntry* ge = work + entry;
  if (m >= ge->count) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, groups = in_dim / 64;
  const float* row = PHASE == 0 ? src + (size_t)(ge->item[m] / top_k) * in_dim : src + (size_t)(entry * MB + m) * 2 * in_dim;
  unsigned char* bdst = xb + (size_t)entry * xb_stride;
  float* tab = xtab + (size_t)entry * tab_stride;
  for (int g = warp; g < groups; g += 8) {
    float v[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int k = g * 64 + h * 32 + lane;
      if (PHASE == 0) {
        v[h] = row[k];
      } else {
        const float gv = row[k], uv = row[in_dim + k];
        v[h] = __fmul_rn(__fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv))), uv);
      }
    }
    // the order of mlx_prep_x_kernel: each half's butterfly, then the halves
    float s0 = v[0], s1 = v[1], mx = fmaxf(fabsf(v[0]), fabsf(v[1]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s0 += __shfl_xor_sync(0xffffffffu, s0, o);
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    const float s = s0 + s1;
    int e = (int)((__float_as_uint(mx) >> 23) & 0xFF);
    if (e < QBITS + 2) e = QBITS + 2;
    if (e > 254) e = 254;
    if (lane == 0) {
      tab[m * groups + g] = s;
      tab[(MB + m) * groups + g] = __uint_as_float((uint32_t)(e - 126 - QBITS + 127) << 23);
    }
    const float fi = __uint_as_float((uint32_t)(QBITS - (e - 126) + 127) << 23);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int q = __float2int_rn(v[h] * fi);
      const int k = (g & 3) * 64 + h * 32 + lane;
      const int step = k >> 5, w = (k & 31) >> 3, j = k & 7;
      const int pos = 8 * w + 4 * (j & 1) + (j >> 1);
      unsigned char* base = bdst + (size_t)(g >> 2) * (N * 256) + step * (N * 32) + (pos >> 4) * ((N / 8) * 128) + (pos & 15);
#pragma unroll
      for (int d = 0; d < DIGITS; ++d) {
        const int dig = d == DIGITS - 1 ? q : ((q + 64) & 127) - 64;
        q = (q - dig) >> 7;
        const int n = m * DIGITS + d;
        base[(n >> 3) * 128 + (n & 7) * 16] = (unsigned char)(dig & 0xFF);
      }
    }
  }
}

bool mlx_mma_grouped_supported(int hidden, int inter) {
  return hidden % kChunkK == 0 && inter % kChunkK == 0 && hidden % kTileRows == 0 && inter % kTileRows == 0 && hidden <= 16384 &&
         inter <= 16384;
}
// four digits per activation row -> 4 * rows accumulator columns
size_t mlx_mma_grouped_xb_bytes(int in_dim, int rows) { return (size_t)(in_dim / kChunkK) * (8 * 4 * rows * 32); }
int mlx_mma_grouped_tab_floats(int in_dim, int rows) { return 2 * rows * (in_dim / 64); }

template <int MB>
static int launch_grouped(int device, const MmaGroupLaunch& g, cudaStream_t stream) {
  constexpr int N = 4 * MB, C = stage_chunks<N, FMT_MLX4>();
  MmaDeviceBufs* bufs = device_bufs(device);
  if (!bufs) return fail(GOPH_E_NOMEM, "cannot allocate the tensor-core path's device scratch");
  DeviceState& st = device_state(device);
  MmaArgs a;
  memset(&a, 0, sizeof a);
  a.status = bufs->status;
  a.xb = g.xb;
  a.xtab = g.xtab;
  a.out = g.out;
  a.out_dim = g.mats * g.rows;
  a.in_dim = g.in_dim;
  a.batch = MB;
  a.ntiles = g.rows / kTileRows;
  a.nchunks = g.in_dim / kChunkK;
  a.splits = 1;
  a.items = g.max_entries * g.mats * a.ntiles;
  a.gwork = g.work;
  a.gcount = g.count;
  a.gmax = g.max_entries;
  a.gtpe = a.ntiles;
  a.gmats = g.mats;
  a.gfirst = g.first;
  a.gdirect = g.phase == 1;
  a.gtab = mlx_mma_grouped_tab_floats(g.in_dim, MB);
  a.gxb = mlx_mma_grouped_xb_bytes(g.in_dim, MB);
  a.dbg = g_mma_dbg;
  size_t fixed = MmaSmem<N, FMT_MLX4, false, C>::bytes(0, MB, g.in_dim);
  int stages = fixed < kMmaSmemBudget ? (int)((kMmaSmemBudget - fixed) / MmaSmem<N, FMT_MLX4, false, C>::kStage) : 0;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 3) return fail(GOPH_E_UNSUPPORTED, "tensor-core experts: %d columns leave no room for the ring", g.in_dim);
  a.stages = stages;
  size_t smem = MmaSmem<N, FMT_MLX4, false, C>::bytes(stages, MB, g.in_dim);
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(g.max_entries * MB);
  cfg.blockDim = dim3(256);
  note_launch();
  if (g.phase == 0)
    GOPH_CUDA(cudaLaunchKernelEx(&cfg, moe_mma_prep_kernel<N, MB, 0>, g.work, g.count, g.max_entries, g.src, g.in_dim, g.top_k, g.xb,
                                 a.gxb, g.xtab, a.gtab));
  else
    GOPH_CUDA(cudaLaunchKernelEx(&cfg, moe_mma_prep_kernel<N, MB, 1>, g.work, g.count, g.max_entries, g.src, g.in_dim, g.top_k, g.xb,
                                 a.gxb, g.xtab, a.gtab));
  auto kern = mlx_mma_kernel<N, 4, MB, FMT_MLX4, false, C, true>;
  GOPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cfg.gridDim = dim3(a.items < st.sm_count ? a.items : st.sm_count);
  cfg.blockDim = dim3(mma_threads<N, FMT_MLX4>());
  cfg.dynamicSmemBytes = smem;
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  return GOPH_OK;
}

int mlx_mma_launch_grouped(int device, const MmaGroupLaunch& g, cudaStream_t stream) {
  if (g.entry_rows == 2) return launch_grouped<2>(device, g, stream);
  if (g.entry_rows == 4) return launch_grouped<4>(device, g, stream);
  return fail(GOPH_E_INVALID, "grouped launch: entries of %d items", g.entry_rows);
}

// ---- GGUF Q4_K / Q8_0 in the tiled layouts ------------------------------------------------------

// Device super-blocks {16-byte header, 8 x 16 bytes of nibbles} -> tiled stages; one thread per 16-byte unit.
__global__ void q4k_tile_kernel(const unsigned char* __restrict__ blocks, unsigned char* __restrict__ tiled, int out_dim,
                                int ntiles, int nchunks) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t nstages = (size_t)ntiles * nchunks;
  if (idx >= nstages * (128 * 9)) return;
  size_t stg = idx / (128 * 9);
  int rem = (int)(idx - stg * (128 * 9));
  int tile = (int)(stg / nchunks), chunk = (int)(stg - (size_t)tile * nchunks);
  int r = rem / 9, u = rem - r * 9;
  int row = tile * 128 + r;
  uint4 v = make_uint4(0, 0, 0, 0);
  unsigned char* dst = tiled + stg * Fmt<FMT_Q4K>::kStageBytes;
  const unsigned char* src = blocks + ((size_t)row * nchunks + chunk) * 144;
  if (u < 8) {
    if (row < out_dim) v = *reinterpret_cast<const uint4*>(src + 16 + 16 * u);
    *reinterpret_cast<uint4*>(dst + r * 128 + ((u ^ (r & 7)) << 4)) = v;
  } else {
    if (row < out_dim) v = *reinterpret_cast<const uint4*>(src);
    *reinterpret_cast<uint4*>(dst + Fmt<FMT_Q4K>::kStageWBytes + r * 16) = v;
  }
}

// Byte plane (q + 128) and f16 scales -> tiled stages of signed bytes; one thread per 16-byte half block.
__global__ void q80_tile_kernel(const unsigned char* __restrict__ plane, const uint16_t* __restrict__ d16,
                                unsigned char* __restrict__ tiled, int out_dim, int in_dim, int ntiles, int nchunks) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t nstages = (size_t)ntiles * nchunks;
  if (idx >= nstages * (128 * 16)) return;
  size_t stg = idx / (128 * 16);
  int rem = (int)(idx - stg * (128 * 16));
  int tile = (int)(stg / nchunks), chunk = (int)(stg - (size_t)tile * nchunks);
  int r = rem >> 4, hb = rem & 15, step = hb >> 1, half = hb & 1;
  int row = tile * 128 + r;
  unsigned char* dst = tiled + stg * Fmt<FMT_Q80>::kStageBytes;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (row < out_dim) {
    v = *reinterpret_cast<const uint4*>(plane + (size_t)row * in_dim + chunk * 256 + step * 32 + half * 16);
    v.x ^= 0x80808080u;
    v.y ^= 0x80808080u;
    v.z ^= 0x80808080u;
    v.w ^= 0x80808080u;
  }
  *reinterpret_cast<uint4*>(dst + step * 4096 + half * 2048 + (r >> 3) * 128 + (r & 7) * 16) = v;
  if (half == 0) {
    uint16_t d = row < out_dim ? d16[(size_t)row * (in_dim / 32) + chunk * 8 + step] : (uint16_t)0;
    *reinterpret_cast<uint16_t*>(dst + Fmt<FMT_Q80>::kStageWBytes + r * 16 + step * 2) = d;
  }
}

// dequantRowQ4KTo / dequantRowQ8_0To from the tiled layouts (loader/gguf/quant_matrix.go:138-158, :281-329).
__global__ void q4k_dequant_tiled_kernel(const unsigned char* __restrict__ tiled, float* __restrict__ out, int out_dim,
                                         int in_dim, int nchunks) {
  size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // 32-element unit of the row-major result
  size_t units_per_row = in_dim / 32;
  if (u >= (size_t)out_dim * units_per_row) return;
  int row = (int)(u / units_per_row), unit = (int)(u - (size_t)row * units_per_row);
  int chunk = unit >> 3, sblk = unit & 7, r = row & 127;
  const unsigned char* stg = tiled + ((size_t)(row >> 7) * nchunks + chunk) * Fmt<FMT_Q4K>::kStageBytes;
  uint4 h = *reinterpret_cast<const uint4*>(stg + Fmt<FMT_Q4K>::kStageWBytes + r * 16);
  uint4 q = *reinterpret_cast<const uint4*>(stg + r * 128 + ((sblk ^ (r & 7)) << 4));
  int bit = 12 * sblk, wi = bit >> 5, sh = bit & 31;
  uint32_t lo = wi == 0 ? h.y : wi == 1 ? h.z : h.w, hi = wi == 0 ? h.z : wi == 1 ? h.w : 0u;
  uint32_t f = __funnelshift_r(lo, hi, sh) & 0xFFFu;
  float sd = __fmul_rn((float)(f & 63u), __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu))));
  float md = __fmul_rn((float)(f >> 6), __half2float(__ushort_as_half((unsigned short)(h.x >> 16))));
  float4* o = reinterpret_cast<float4*>(out + u * 32);
  uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __fsub_rn(__fmul_rn(sd, (float)((ws[k] >> (4 * e)) & 0xF)), md);
    o[2 * k] = make_float4(v[0], v[1], v[2], v[3]);
    o[2 * k + 1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

__global__ void q80_dequant_tiled_kernel(const unsigned char* __restrict__ tiled, float* __restrict__ out, int out_dim,
                                         int in_dim, int nchunks) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)out_dim * in_dim) return;
  int row = (int)(i / in_dim), col = (int)(i - (size_t)row * in_dim);
  int chunk = col >> 8, k = col & 255, step = k >> 5, half = (k >> 4) & 1, r = row & 127;
  const unsigned char* stg = tiled + ((size_t)(row >> 7) * nchunks + chunk) * Fmt<FMT_Q80>::kStageBytes;
  signed char q = (signed char)stg[step * 4096 + half * 2048 + (r >> 3) * 128 + (r & 7) * 16 + (k & 15)];
  uint16_t d = *reinterpret_cast<const uint16_t*>(stg + Fmt<FMT_Q80>::kStageWBytes + r * 16 + step * 2);
  out[i] = __fmul_rn(__half2float(__ushort_as_half(d)), (float)q);
}

// Q5_K super-blocks in the streaming layout {16-byte header, 8 x 16 bytes of nibbles, 8 x 4 bytes of
// fifth bits} -> stages of unsigned bytes in Q80's order + the header; one thread per 16-byte unit.
__global__ void q5k_tile_kernel(const unsigned char* __restrict__ blocks, unsigned char* __restrict__ tiled, int out_dim,
                                int ntiles, int nchunks) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t nstages = (size_t)ntiles * nchunks;
  if (idx >= nstages * (128 * 17)) return;
  size_t stg = idx / (128 * 17);
  int rem = (int)(idx - stg * (128 * 17));
  int tile = (int)(stg / nchunks), chunk = (int)(stg - (size_t)tile * nchunks);
  int r = rem / 17, hb = rem - r * 17, row = tile * 128 + r;
  unsigned char* dst = tiled + stg * Fmt<FMT_Q5K>::kStageBytes;
  const unsigned char* src = blocks + ((size_t)row * nchunks + chunk) * 176;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (hb == 16) {
    if (row < out_dim) v = *reinterpret_cast<const uint4*>(src);
    *reinterpret_cast<uint4*>(dst + Fmt<FMT_Q5K>::kStageWBytes + r * 16) = v;
    return;
  }
  const int step = hb >> 1, half = hb & 1;
  if (row < out_dim) {
    const uint2 q = *reinterpret_cast<const uint2*>(src + 16 + 16 * step + 8 * half);  // 16 nibbles
    const uint32_t fifth = *reinterpret_cast<const uint32_t*>(src + 144 + 4 * step) >> (16 * half);
    uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t nib = ((j < 8 ? q.x : q.y) >> (4 * (j & 7))) & 0xFu;
      out[j >> 2] |= (nib | (((fifth >> j) & 1u) << 4)) << (8 * (j & 3));
    }
    v = make_uint4(out[0], out[1], out[2], out[3]);
  }
  *reinterpret_cast<uint4*>(dst + step * 4096 + half * 2048 + (r >> 3) * 128 + (r & 7) * 16) = v;
}

// Q6_K planes (low nibbles, two-bit highs, int8 scales, f16 d) -> stages of signed bytes (value - 32)
// in Q80's order + {16 scales, d, padding} per row; one thread per 16-byte unit.
__global__ void q6k_tile_kernel(const unsigned char* __restrict__ lo, const unsigned char* __restrict__ hi,
                                const signed char* __restrict__ sc, const uint16_t* __restrict__ dd,
                                unsigned char* __restrict__ tiled, int out_dim, int in_dim, int ntiles, int nchunks) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t nstages = (size_t)ntiles * nchunks;
  if (idx >= nstages * (128 * 18)) return;
  size_t stg = idx / (128 * 18);
  int rem = (int)(idx - stg * (128 * 18));
  int tile = (int)(stg / nchunks), chunk = (int)(stg - (size_t)tile * nchunks);
  int r = rem / 18, hb = rem - r * 18, row = tile * 128 + r;
  unsigned char* dst = tiled + stg * Fmt<FMT_Q6K>::kStageBytes;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (hb == 16) {
    if (row < out_dim) v = *reinterpret_cast<const uint4*>(sc + (size_t)row * (in_dim / 16) + chunk * 16);
    *reinterpret_cast<uint4*>(dst + Fmt<FMT_Q6K>::kStageWBytes + r * 32) = v;
    return;
  }
  if (hb == 17) {
    if (row < out_dim) v.x = dd[(size_t)row * nchunks + chunk];
    *reinterpret_cast<uint4*>(dst + Fmt<FMT_Q6K>::kStageWBytes + r * 32 + 16) = v;
    return;
  }
  const int step = hb >> 1, half = hb & 1;
  if (row < out_dim) {
    const size_t col = (size_t)chunk * 256 + step * 32 + half * 16;  // 16 elements: two words of nibbles, one of highs
    const uint2 wl = *reinterpret_cast<const uint2*>(lo + (size_t)row * (in_dim / 2) + col / 2);
    const uint32_t wh = *reinterpret_cast<const uint32_t*>(hi + (size_t)row * (in_dim / 4) + col / 4);
    uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = (int)((((j < 8 ? wl.x : wl.y) >> (4 * (j & 7))) & 0xFu) | (((wh >> (2 * j)) & 3u) << 4)) - 32;
      out[j >> 2] |= (uint32_t)(q & 0xFF) << (8 * (j & 3));
    }
    v = make_uint4(out[0], out[1], out[2], out[3]);
  }
  *reinterpret_cast<uint4*>(dst + step * 4096 + half * 2048 + (r >> 3) * 128 + (r & 7) * 16) = v;
}

// dequantRowQ5K / dequantRowQ6K from the tiled layouts (loader/gguf/quant_matrix.go:331-426), the
// roundings of the streaming layouts' kernels.
__global__ void q5k_dequant_tiled_kernel(const unsigned char* __restrict__ tiled, float* __restrict__ out, int out_dim,
                                         int in_dim, int nchunks) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)out_dim * in_dim) return;
  int row = (int)(i / in_dim), col = (int)(i - (size_t)row * in_dim);
  int chunk = col >> 8, k = col & 255, step = k >> 5, half = (k >> 4) & 1, r = row & 127;
  const unsigned char* stg = tiled + ((size_t)(row >> 7) * nchunks + chunk) * Fmt<FMT_Q5K>::kStageBytes;
  const uint4 h = *reinterpret_cast<const uint4*>(stg + Fmt<FMT_Q5K>::kStageWBytes + r * 16);
  const int bit = 12 * step, wi = bit >> 5, sh = bit & 31;
  const uint32_t lo = wi == 0 ? h.y : wi == 1 ? h.z : h.w, hi = wi == 0 ? h.z : wi == 1 ? h.w : 0u;
  const uint32_t f = __funnelshift_r(lo, hi, sh) & 0xFFFu;
  const float sd = __fmul_rn((float)(f & 63u), __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu))));
  const float md = __fmul_rn((float)(f >> 6), __half2float(__ushort_as_half((unsigned short)(h.x >> 16))));
  const unsigned char q = stg[step * 4096 + half * 2048 + (r >> 3) * 128 + (r & 7) * 16 + (k & 15)];
  out[i] = __fsub_rn(__fmul_rn(sd, (float)q), md);
}

__global__ void q6k_dequant_tiled_kernel(const unsigned char* __restrict__ tiled, float* __restrict__ out, int out_dim,
                                         int in_dim, int nchunks) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)out_dim * in_dim) return;
  int row = (int)(i / in_dim), col = (int)(i - (size_t)row * in_dim);
  int chunk = col >> 8, k = col & 255, step = k >> 5, half = (k >> 4) & 1, r = row & 127;
  const unsigned char* stg = tiled + ((size_t)(row >> 7) * nchunks + chunk) * Fmt<FMT_Q6K>::kStageBytes;
  const unsigned char* mrow = stg + Fmt<FMT_Q6K>::kStageWBytes + r * 32;
  const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(mrow + 16)));
  const signed char sc = (signed char)mrow[k >> 4];
  const signed char q = (signed char)stg[step * 4096 + half * 2048 + (r >> 3) * 128 + (r & 7) * 16 + (k & 15)];
  out[i] = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
}

bool gguf_mma_supported(int qtype, int in_dim) {
  return (qtype == GOPH_GGUF_Q4_K || qtype == GOPH_GGUF_Q8_0 || qtype == GOPH_GGUF_Q5_K || qtype == GOPH_GGUF_Q6_K) &&
         in_dim % kChunkK == 0 && in_dim <= kMaxPrepIn;
}

int gguf_mma_make_tiled(goph_gguf_matrix* m) {
  const int ntiles = (m->out_dim + kTileRows - 1) / kTileRows, nchunks = m->in_dim / kChunkK;
  const bool q4 = m->qtype == GOPH_GGUF_Q4_K;
  const size_t stage = q4 ? Fmt<FMT_Q4K>::kStageBytes
                          : m->qtype == GOPH_GGUF_Q5_K ? Fmt<FMT_Q5K>::kStageBytes
                          : m->qtype == GOPH_GGUF_Q6_K ? Fmt<FMT_Q6K>::kStageBytes : Fmt<FMT_Q80>::kStageBytes;
  const size_t bytes = (size_t)ntiles * nchunks * stage;
  unsigned char* t = nullptr;
  GOPH_CUDA(cudaMalloc(&t, bytes));
  if (q4) {
    size_t threads = (size_t)ntiles * nchunks * 128 * 9;
    q4k_tile_kernel<<<(unsigned)((threads + 255) / 256), 256>>>(m->data, t, m->out_dim, ntiles, nchunks);
  } else if (m->qtype == GOPH_GGUF_Q5_K) {
    size_t threads = (size_t)ntiles * nchunks * 128 * 17;
    q5k_tile_kernel<<<(unsigned)((threads + 255) / 256), 256>>>(m->data, t, m->out_dim, ntiles, nchunks);
  } else if (m->qtype == GOPH_GGUF_Q6_K) {
    // planes behind one another: low nibbles in data; highs, int8 scales, f16 d in d16's buffer
    const size_t n = (size_t)m->out_dim * m->in_dim;
    const unsigned char* hi = reinterpret_cast<const unsigned char*>(m->d16);
    size_t threads = (size_t)ntiles * nchunks * 128 * 18;
    q6k_tile_kernel<<<(unsigned)((threads + 255) / 256), 256>>>(m->data, hi, reinterpret_cast<const signed char*>(hi + n / 4),
                                                                reinterpret_cast<const uint16_t*>(hi + n / 4 + n / 16), t, m->out_dim,
                                                                m->in_dim, ntiles, nchunks);
  } else {
    size_t threads = (size_t)ntiles * nchunks * 128 * 16;
    q80_tile_kernel<<<(unsigned)((threads + 255) / 256), 256>>>(m->data, m->d16, t, m->out_dim, m->in_dim, ntiles, nchunks);
  }
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(t);
    return fail_cuda(e, "gguf tile kernel");
  }
  m->tiled = t;
  m->bytes = bytes;
  return GOPH_OK;
}

int gguf_mma_launch(const goph_gguf_matrix* m, float* out, const float* x, int batch, int digits, cudaStream_t stream,
                    bool x_prepared) {
  if (!m->tiled) return fail(GOPH_E_UNSUPPORTED, "matrix is not in the tiled layout");
  TiledDesc d{m->tiled, m->device, m->out_dim, m->in_dim};
  if (m->qtype == GOPH_GGUF_Q4_K) return tiled_launch<FMT_Q4K>(d, out, x, batch, digits, stream, x_prepared);
  if (m->qtype == GOPH_GGUF_Q5_K) return tiled_launch<FMT_Q5K>(d, out, x, batch, digits, stream, x_prepared);
  if (m->qtype == GOPH_GGUF_Q6_K) return tiled_launch<FMT_Q6K>(d, out, x, batch, digits, stream, x_prepared);
  return tiled_launch<FMT_Q80>(d, out, x, batch, digits, stream, x_prepared);
}

int gguf_mma_dequant(const goph_gguf_matrix* m, float* out, cudaStream_t stream) {
  const int nchunks = m->in_dim / kChunkK;
  if (m->qtype == GOPH_GGUF_Q4_K) {
    size_t units = (size_t)m->out_dim * (m->in_dim / 32);
    q4k_dequant_tiled_kernel<<<(unsigned)((units + 255) / 256), 256, 0, stream>>>(m->tiled, out, m->out_dim, m->in_dim, nchunks);
  } else if (m->qtype == GOPH_GGUF_Q5_K || m->qtype == GOPH_GGUF_Q6_K) {
    size_t n = (size_t)m->out_dim * m->in_dim;
    if (m->qtype == GOPH_GGUF_Q5_K)
      q5k_dequant_tiled_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(m->tiled, out, m->out_dim, m->in_dim, nchunks);
    else
      q6k_dequant_tiled_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(m->tiled, out, m->out_dim, m->in_dim, nchunks);
  } else {
    size_t n = (size_t)m->out_dim * m->in_dim;
    q80_dequant_tiled_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(m->tiled, out, m->out_dim, m->in_dim, nchunks);
  }
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

// ---- GEMV without any allocation ---------------------------------------------------------------
// Some callers must not allocate device memory when they run a product: a serving loop that has
// handed the whole memory budget to its KV and expert pools (an allocation could fail, or block
// behind a free), a thread that may not take the allocator's device-wide synchronisation in the
// middle of a decode step, or code that has begun capturing a stream.  For them the scratch of the
// tensor-core GEMV (status word, tile counters, the prepared activation digits and tables, the
// split-K partial sums) lives in this file-scope device array instead of in buffers obtained with
// cudaMalloc.  Every GPU that loads the library carries the array until the process exits.
constexpr int kNoAllocMaxIn = 16384;     // largest in_dim the entry point accepts
constexpr int kNoAllocMaxTiles = 4096;   // largest ceil(out_dim / 128)
constexpr int kNoAllocMaxItems = 192;    // (tile, split) items that may have partial sums at once
constexpr size_t kNaStatusOff = 0;
constexpr size_t kNaCountersOff = 256;
constexpr size_t kNaTabOff = kNaCountersOff + (size_t)kNoAllocMaxTiles * 4;
constexpr size_t kNaXbOff = kNaTabOff + (size_t)2 * (kNoAllocMaxIn / 64) * 4;
constexpr size_t kNaPartOff = kNaXbOff + (size_t)8 * kNoAllocMaxIn;
constexpr size_t kNoAllocBytes = kNaPartOff + (size_t)kNoAllocMaxItems * kTileRows * 4;
static_assert(kNaTabOff % 256 == 0 && kNaXbOff % 256 == 0 && kNaPartOff % 256 == 0, "256-byte aligned regions");
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];  // 248,064 bytes

// Device address of the array on `device` (which must be current).  In host code the array's
// name is only a handle for the runtime, never a pointer a kernel could use, so the address is
// looked up once per device with cudaGetSymbolAddress and cached.
static int noalloc_base(int device, unsigned char** base) {
  static unsigned char* cached[kMaxDevices] = {};
  if (!cached[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
    if (!p) return fail(GOPH_E_CUDA, "cudaGetSymbolAddress returned a null address for the scratch array");
    cached[device] = static_cast<unsigned char*>(p);
  }
  *base = cached[device];
  return GOPH_OK;
}

template <int DIGITS>
static int launch_noalloc(const goph_mlx_weight* w, float* out, const float* x, unsigned char* base,
                          cudaStream_t stream) {
  constexpr int N = 8, MB = 1;
  DeviceState& st = device_state(w->device);
  MmaArgs a;
  memset(&a, 0, sizeof a);
  a.w = w->tiled;
  a.x = x;
  a.out = out;
  a.status = reinterpret_cast<int*>(base + kNaStatusOff);
  a.counters = reinterpret_cast<unsigned int*>(base + kNaCountersOff);
  a.xtab = reinterpret_cast<const float*>(base + kNaTabOff);
  a.xb = base + kNaXbOff;
  a.scratch = reinterpret_cast<float*>(base + kNaPartOff);
  a.out_dim = w->out_dim;
  a.in_dim = w->in_dim;
  a.batch = 1;
  a.ntiles = (w->out_dim + kTileRows - 1) / kTileRows;
  a.nchunks = w->in_dim / kChunkK;
  size_t fixed = MmaSmem<N>::bytes(0, 1, a.in_dim);
  int stages = (int)(((size_t)kSmemBudget - fixed) / MmaSmem<N>::kStage);
  if (stages > 8) stages = 8;
  a.stages = stages;
  int splits = 1;
  if (a.ntiles < st.sm_count) {
    splits = st.sm_count / a.ntiles;
    if (splits > a.nchunks) splits = a.nchunks;
    if (splits < 1) splits = 1;
  }
  while (splits > 1 && a.ntiles * splits > kNoAllocMaxItems) --splits;
  a.splits = splits;
  a.items = a.ntiles * splits;
  a.cmax = 0;
  // The array keeps whatever the last call left: the tile counters have to start at zero (the
  // digits, tables and partial sums are fully rewritten before they are read).  The status word is
  // left alone: it is zero when the library is loaded and sticky once a wait has given up, like the
  // allocated path's; goph_mlx_gemv_noalloc_status reads it.
  GOPH_CUDA(cudaMemsetAsync(base + kNaCountersOff, 0, kNaTabOff - kNaCountersOff, stream));
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 0;  // plain stream order behind the memset
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(a.in_dim / 64);
  cfg.blockDim = dim3(64);
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, mlx_prep_x_kernel<DIGITS>, a.x, const_cast<unsigned char*>(a.xb),
                               const_cast<float*>(a.xtab), 1, a.in_dim, N));
  size_t smem = MmaSmem<N>::bytes(stages, 1, a.in_dim);
  if (smem < 120 * 1024) smem = 120 * 1024;
  auto kern = mlx_mma_kernel<N, DIGITS, MB>;
  GOPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cfg.gridDim = dim3(a.items < st.sm_count ? a.items : st.sm_count);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  return GOPH_OK;
}

}  // namespace goph

using namespace goph;

#ifdef GOPH_TUNING
GOPH_API int goph_tuning_set_gemv(int dbg) {
  goph::g_mma_dbg = dbg;
  return 0;
}
GOPH_API int goph_tuning_probe_gemv(long long* out512) {
  return cudaMemcpyFromSymbol(out512, g_mma_trace, 8 * 64 * sizeof(long long)) == cudaSuccess ? 0 : -1;
}
#endif

GOPH_API int goph_mlx_gemv_noalloc_status(int device, int* out_status) {
  clear_error();
  if (!out_status) return fail(GOPH_E_INVALID, "goph_mlx_gemv_noalloc_status: nil result pointer");
  if (int rc = use_device(device)) return rc;
  unsigned char* base = nullptr;
  if (int rc = noalloc_base(device, &base)) return rc;
  GOPH_CUDA(cudaMemcpy(out_status, base + kNaStatusOff, sizeof(int), cudaMemcpyDeviceToHost));
  return GOPH_OK;
}

GOPH_API int goph_mlx_gemv_noalloc(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                                   const goph_mlx_weight* w, void* stream) {
  clear_error();
  if (!w || w->magic != kMagicMLX) return fail(GOPH_E_INVALID, "invalid MLX weight handle");
  if (!w->tiled)
    return fail(GOPH_E_UNSUPPORTED,
                "goph_mlx_gemv_noalloc needs a weight in the tiled layout (group size 64, in_dim a multiple of 256, "
                "uploaded with mlx_layout 0 or 2); this one is row-major");
  if (w->in_dim > kNoAllocMaxIn)
    return fail(GOPH_E_UNSUPPORTED, "goph_mlx_gemv_noalloc: in_dim=%d is above the built-in scratch limit of %d", w->in_dim,
                kNoAllocMaxIn);
  if ((w->out_dim + kTileRows - 1) / kTileRows > kNoAllocMaxTiles)
    return fail(GOPH_E_UNSUPPORTED, "goph_mlx_gemv_noalloc: out_dim=%d is above the built-in scratch limit of %d", w->out_dim,
                kNoAllocMaxTiles * kTileRows);
  if (!x_dev || x_len < (uint64_t)w->in_dim || !out_dev || out_len < (uint64_t)w->out_dim)
    return fail(GOPH_E_INVALID, "buffers x=%llu/%d out=%llu/%d", (unsigned long long)x_len, w->in_dim,
                (unsigned long long)out_len, w->out_dim);
  if ((uintptr_t)x_dev % 16) return fail(GOPH_E_INVALID, "goph_mlx_gemv_noalloc: x must be 16-byte aligned");
  if (int rc = use_device(w->device)) return rc;
  unsigned char* base = nullptr;
  if (int rc = noalloc_base(w->device, &base)) return rc;
  return options().mlx_digits == 3 ? launch_noalloc<3>(w, out_dev, x_dev, base, (cudaStream_t)stream)
                                   : launch_noalloc<4>(w, out_dev, x_dev, base, (cudaStream_t)stream);
}
