// FP8 E4M3 linears on the 5th-generation tensor cores with nothing converted on the way:
// tcgen05.mma kind::f8f6f4, both operands read from shared memory through descriptors, f32
// accumulators in TMEM.  One kernel for every batch size of a linear in the tensor-core layout.
//
// Stands behind nvidia.GemvFP8E4M3Buffer / GemmFP8E4M3Buffer (backends/nvidia/runtime/fp8.go:158-222,
// :271-320; kernel text backends/nvidia/ptx/fp8/fp8.go:154-309, which decodes every weight on the
// CUDA cores and re-reads the weights for every batch row).
//
// Arithmetic
//   * A operand (weights, M = 128 rows of a tile): the e4m3 bytes as they lie in the checkpoint.  The
//     tensor core decodes normals and subnormals exactly.  (A linear that contains one of the two NaN
//     codes keeps the row-major layout and the CUDA-core kernel, which reproduces the NaN.)
//   * B operand (activations): each activation row is scaled by a power of two so that its largest
//     magnitude lies in [128, 256) and every element is written as the sum of P e4m3 values, each
//     the truncation of what the pieces before it left over; after every second piece the remainder
//     is multiplied by 2^8 (and the piece's accumulator column by 2^-8 in the epilogue), which keeps
//     it inside e4m3's narrow range (smallest subnormal 2^-9).  P = 2 holds a bf16 value exactly
//     down to 2^-17 of the row's largest element, P = 4 holds 16 significant bits, P = 6 an f32
//     exactly.  Piece p of row m is B row p * MP + m.
//   * Every product of two e4m3 values is exact in f32; the tensor core accumulates in f32 over the
//     whole K range of an item, so there is one epilogue per (tile, K split), not per stage.
//   * Epilogue: out[m][r] = (sum over pieces of D[r][p * MP + m]) * 2^-e(m) * scale[r] + bias[r]
//     (fp8.Linear.GemvTo, backends/simd/quant/fp8/fp8.go:219-239).
//
// Device layout of the weights (built at upload): blocks of 128 rows x 256 bytes ordered
// [row tile][K chunk]; inside a block the K-major 8 x 16-byte core matrices the MMA reads:
// [K step of 32 (8)][K half of 16 (2)][row group (16)][row (8)][16 B].  A block, or half a block (128
// rows x 128 bytes of K) where the B tile is wide, is one pipeline stage and one contiguous bulk copy.
//
// Pipeline of one CTA (10 warps, one persistent CTA per SM, walking (tile, K split) items):
//   producer warp   per stage one bulk copy of the weights and one of the B tile into a ring guarded by full/empty mbarriers; the weight copies of the first two
//                   stages are issued before the kernel in front (the activation preparation) ends.
//   MMA warp        waits as a warp, one elected lane issues the stage's M128 x N x K32 instructions
//                   (eight, or four) and commits to the stage's barrier and, after an item's last stage, to the
//                   accumulator's.  Two accumulator buffers: the next item's MMAs run while the
//                   epilogue reads the last one.
//   8 epilogue warps  two per TMEM lane quarter, each with half of the activation rows: tcgen05.ld,
//                   pieces added, scales, store; K splits go through scratch and the CTA that arrives
//                   last at the tile adds them in split order.
// Every wait is bounded (~2 s); a waiter that gives up records a code (500+) in the status word and
// the CTA winds down.
#include <string.h>

#include <mutex>

#include "goph_internal.cuh"
#include "tc_common.cuh"
#include "tc_gemm.cuh"

namespace goph {

using namespace tc;

namespace {

constexpr int kTileRows = 128;
constexpr int kChunkK = 256;                          // a block of the layout
constexpr int kBlockBytes = kTileRows * kChunkK;      // 32 KiB
constexpr int kThreads = 10 * 32;
constexpr int kEpiWarps = 8, kEpiThreads = kEpiWarps * 32;
constexpr int kMaxStages = 10;
constexpr int kMaxIn = 65536;
constexpr size_t kXbBytes = (size_t)256 * kMaxIn;     // 256 B rows of up to kMaxIn bytes
constexpr int kMaxItems = 320;
constexpr size_t kScratchFloats = (size_t)kMaxItems * 64 * kTileRows;
constexpr size_t kMaxCounters = 4096;
constexpr size_t kSmemBudget = 222 * 1024;
constexpr int kPrepSlice = 4096;                      // elements of a row one preparation CTA converts
constexpr int kRecvBytes = 16 * 1024;                 // cluster launches: partial sums the first CTA of a cluster can receive

struct Fp8Args {
  const unsigned char* w;   // tiled weight blocks [tile][chunk]
  const unsigned char* xb;  // B tiles [chunk][K step 8][K half 2][N/8][8 rows][16 B]
  const float* xinv;        // [MP] 2^-e of the activation rows
  const float* scale;       // [out_dim]
  const float* bias;        // [out_dim] or nullptr
  float* out;               // [batch][out_dim]
  int* status;
  float* scratch;           // split-K partial sums [tile][split][MP][128]
  unsigned int* counters;   // per-tile arrival counters, zero between launches
  int out_dim, in_dim, batch;
  int ntiles, nks, splits, items, stages;  // nks: stages along K (in_dim / KS); items = row-tile groups x splits
  // 1: the K splits of a group are the CTAs of a thread-block cluster (every CTA has one item) and
  // their partial sums go through the first CTA's shared memory instead of device scratch
  int cluster;
};

struct ItemWalk {
  int w, tile, split, k, k1;  // tile: the item's group of TT consecutive row tiles
  __device__ __forceinline__ void open(const Fp8Args& a) {
    tile = w / a.splits;
    split = w - tile * a.splits;
    k = split * a.nks / a.splits;
    k1 = (split + 1) * a.nks / a.splits;
  }
  __device__ __forceinline__ ItemWalk(const Fp8Args& a) : w(blockIdx.x) {
    if (w < a.items) open(a);
  }
  __device__ __forceinline__ bool live(const Fp8Args& a) const { return w < a.items; }
  __device__ __forceinline__ bool last_stage() const { return k + 1 == k1; }
  __device__ __forceinline__ void next(const Fp8Args& a) {
    if (++k == k1) {
      w += gridDim.x;
      if (w < a.items) open(a);
    }
  }
};

// ---- activation preparation -------------------------------------------------------------------

// Largest e4m3 value of the same sign whose magnitude does not exceed |v| (|v| < 512), and what it
// is worth.  Normals: exponent -6..8, three mantissa bits; subnormals: multiples of 2^-9.
__device__ __forceinline__ uint32_t e4m3_trunc(float v, float* worth) {
  const uint32_t b = __float_as_uint(v), sign = (b >> 24) & 0x80u, a = b & 0x7FFFFFFFu;
  const int e = (int)(a >> 23) - 127;
  if (e < -9) {
    *worth = 0.f;
    return 0u;
  }
  if (e < -6) {
    const uint32_t q = (uint32_t)(__uint_as_float(a) * 512.f);  // 1..7
    *worth = __uint_as_float((b & 0x80000000u) | __float_as_uint((float)q * 0.001953125f));
    return sign | q;
  }
  const uint32_t kept = a & 0xFFF00000u;  // sign-less value with three mantissa bits
  *worth = __uint_as_float((b & 0x80000000u) | kept);
  return sign | (((uint32_t)(e + 7) << 3) & 0x78u) | ((a >> 20) & 7u);  // (the mask only matters for inf / NaN in x)
}

// One CTA per B row group member m (activation row): the row's largest magnitude, then 16 elements
// per thread and step -> one 16-byte core-matrix row per piece.  Rows past `batch` are zeros.
template <int P, bool XBF16>
__global__ void __launch_bounds__(256)
fp8_prep_x_kernel(const void* __restrict__ xv, unsigned char* __restrict__ xb, float* __restrict__ xinv, int batch, int in_dim,
                  int N, int MP) {
  __shared__ float red[8];
  const int m = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();  // x may be the output of the kernel in front; the tiles may still be read by it
  const bool real = m < batch;
  float mx = 0.f;
  if (real) {
    for (int k = tid * 8; k < in_dim; k += 256 * 8) {
      float v[8];
      if (XBF16) {
        const uint4 q = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(xv) + (size_t)m * in_dim + k);
        const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[2 * j] = __uint_as_float(ws[j] << 16);
          v[2 * j + 1] = __uint_as_float(ws[j] & 0xFFFF0000u);
        }
      } else {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(xv) + (size_t)m * in_dim + k);
        const float4 c = p[0], d = p[1];
        v[0] = c.x; v[1] = c.y; v[2] = c.z; v[3] = c.w;
        v[4] = d.x; v[5] = d.y; v[6] = d.z; v[7] = d.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(v[j]));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
  // scale 2^(7 - E), E the exponent of the largest magnitude: the largest element lands in [128, 256)
  int E = (int)((__float_as_uint(mx) >> 23) & 0xFFu) - 127;
  if (mx == 0.f || E > 127) E = 7;          // an all-zero row, or inf / NaN in x (whose products are not finite anyway)
  if (E < -119) E = -119;                   // keeps 2^(7 - E) a normal float
  const float s = __uint_as_float((uint32_t)(7 - E + 127) << 23);
  if (tid == 0 && blockIdx.y == 0) xinv[m] = __uint_as_float((uint32_t)(E - 7 + 127) << 23);
  // every CTA of a row finds the row's largest magnitude for itself (the row comes from the L2);
  // the conversion is shared out in slices of K
  const int k_end = (int)(blockIdx.y + 1) * kPrepSlice < in_dim ? (int)(blockIdx.y + 1) * kPrepSlice : in_dim;
  for (int k = blockIdx.y * kPrepSlice + tid * 16; k < k_end; k += 256 * 16) {
    float v[16];
    if (real) {
      if (XBF16) {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(xv) + (size_t)m * in_dim + k);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 q = p[h];
          const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[8 * h + 2 * j] = __uint_as_float(ws[j] << 16) * s;
            v[8 * h + 2 * j + 1] = __uint_as_float(ws[j] & 0xFFFF0000u) * s;
          }
        }
      } else {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(xv) + (size_t)m * in_dim + k);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float4 c = p[h];
          v[4 * h] = c.x * s; v[4 * h + 1] = c.y * s; v[4 * h + 2] = c.z * s; v[4 * h + 3] = c.w * s;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = 0.f;
    }
    const int chunk = k >> 8, step = (k & 255) >> 5, half = (k & 31) >> 4;
    unsigned char* dst = xb + (size_t)chunk * (N * 256) + step * (N * 32) + half * ((N / 8) * 128);
#pragma unroll
    for (int p = 0; p < P; ++p) {
      uint32_t words[4] = {0, 0, 0, 0};
      if (p > 0 && (p & 1) == 0) {  // every second piece: what is left moves up by 2^8, back into e4m3's range
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= 256.f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float worth;
        const uint32_t code = e4m3_trunc(v[j], &worth);
        v[j] -= worth;  // exact: the remainder of a truncation fits f32
        words[j >> 2] |= code << (8 * (j & 3));
      }
      const int n = p * MP + m;
      *reinterpret_cast<uint4*>(dst + (n >> 3) * 128 + (n & 7) * 16) = make_uint4(words[0], words[1], words[2], words[3]);
    }
  }
}

// G (1, 2, 4, 8 or 16) consecutive accumulator columns of this warp's 32 lanes.
template <int G>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&t)[G]) {
  static_assert(G == 1 || G == 2 || G == 4 || G == 8 || G == 16, "1..16 columns");
  if constexpr (G == 1) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(t[0]) : "r"(taddr) : "memory");
  } else if constexpr (G == 2) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(t[0]), "=r"(t[1]) : "r"(taddr) : "memory");
  } else if constexpr (G == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(t[0]), "=r"(t[1]), "=r"(t[2]), "=r"(t[3])
                 : "r"(taddr)
                 : "memory");
  } else if constexpr (G == 8) {
    tmem_ld8(taddr, t);
  } else {
    tmem_ld16(taddr, t);
  }
}
template <int G>
__device__ __forceinline__ void tmem_ld_cols_wait(uint32_t (&t)[G]) {
  if constexpr (G == 1) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(t[0]) : : "memory");
  } else if constexpr (G == 2) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(t[0]), "+r"(t[1]) : : "memory");
  } else if constexpr (G == 4) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]) : : "memory");
  } else {
    tmem_wait_ld(t);
  }
}

// D[tmem] (+)= A[smem descriptor] * B[smem descriptor], e4m3 operands, f32 accumulate.
__device__ __forceinline__ void umma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// ---- the product kernel -----------------------------------------------------------------------
// KS: K bytes of a pipeline stage, 256 (a whole block) or 128 (half a block, for wide B tiles).  The
// MMA warp spends some 70 cycles per instruction and 300 per stage on waits and commits, so the
// longer stage is what lets a single SM keep up with its share of the HBM rate.
// TT: row tiles per item (1 or 2).  With a wide B tile (64 activation rows in two pieces are 128 B
// rows: 16 KiB of activations per 16 KiB of weights, re-read from the L2 for every row tile) two row
// tiles share each B tile: half the L2 traffic and twice the MMAs per wait and commit.
template <int N, int P, int MP, int KS, int TT>
__global__ void __launch_bounds__(kThreads, 1)
fp8_mma_kernel(const __grid_constant__ Fp8Args a) {
  static_assert(KS == 128 || KS == 256, "a stage is a block or half a block");
  static_assert(TT == 1 || (TT == 2 && 4 * N <= 512), "two accumulator buffers of TT x N columns");
  constexpr int kABytes = kTileRows * KS;
  static_assert(N % 16 == 0 && N >= 16 && N <= 256 && P * MP <= N, "B rows: P pieces of MP activation rows (the rows past P * MP are unused)");
  constexpr int HM = MP / 2;           // rows of one epilogue warp
  constexpr int G = HM >= 16 ? 16 : HM;  // rows per register group
  static_assert(MP >= 2 && MP % 2 == 0 && HM % G == 0, "rows split over two epilogue warps in groups");
  constexpr int kBBytes = N * KS;
  constexpr int kStage = TT * kABytes + kBBytes;  // [TT weight tiles][B tile]
  constexpr int ND = 2;                // accumulator buffers of TT x N columns
  constexpr float kPieceScale[3] = {1.f, 1.f / 256.f, 1.f / 65536.f};  // pieces 2p and 2p+1 were written 2^(8p) up
  constexpr uint32_t kCols = 512;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  const int S = a.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)S * kStage);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 2 * ND + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* recv = reinterpret_cast<float*>(tmem_holder + 4);  // cluster launches: [split - 1][tile of the group][row m][128]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * S, dfull0 = empty0 + 8 * S, dfree0 = dfull0 + 8 * ND;
  const uint32_t clbar = dfree0 + 8 * ND;  // cluster launches: the other CTAs' partial sums have arrived (one arrival per epilogue warp)

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < ND; ++b) {
      mbar_init(dfull0 + 8 * b, 1);
      mbar_init(dfree0 + 8 * b, kEpiWarps);
    }
    if (a.cluster) mbar_init(clbar, kEpiWarps * (a.splits - 1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_launch_dependents();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (a.cluster) cluster_sync_all();  // the first CTA's barrier is initialised before any peer can arrive on it
  const uint32_t tmem_base = *tmem_holder;
  bool ok = true;
  ItemWalk wk(a);
  const int nchunks = a.in_dim / kChunkK;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      auto a_src = [&](const ItemWalk& q, int t) {
        const size_t tile = (size_t)q.tile * TT + t;
        return KS == 256 ? a.w + (tile * nchunks + q.k) * kBlockBytes : a.w + (tile * nchunks + (q.k >> 1)) * kBlockBytes + (q.k & 1) * kABytes;
      };
      // row tiles of the item that exist (the last group of an odd tile count has one)
      auto tiles_of = [&](const ItemWalk& q) { return q.tile * TT + TT <= a.ntiles ? TT : a.ntiles - q.tile * TT; };
      auto b_src = [&](const ItemWalk& q) {
        return KS == 256 ? a.xb + (size_t)q.k * (N * kChunkK) : a.xb + (size_t)(q.k >> 1) * (N * kChunkK) + (q.k & 1) * kBBytes;
      };
      int i = 0;
      {
        // the weights do not depend on the kernel in front: the first stages' copies go out at once
        ItemWalk q = wk;
        for (; i < S && i < 2 && q.live(a); ++i, q.next(a)) {
          const int nt = tiles_of(q);
          mbar_expect_tx(full0 + 8 * i, nt * kABytes + kBBytes);
          for (int t = 0; t < nt; ++t)
            bulk_load_1d(smem_u32(ring + (size_t)i * kStage) + t * kABytes, a_src(q, t), kABytes, full0 + 8 * i);
        }
        pdl_wait();
        for (int j = 0; j < i; ++j, wk.next(a))
          bulk_load_1d(smem_u32(ring + (size_t)j * kStage) + TT * kABytes, b_src(wk), kBBytes, full0 + 8 * j);
      }
      for (; wk.live(a) && ok; ++i, wk.next(a)) {
        const int slot = i % S, round = i / S;
        if (round > 0) ok = mbar_wait(empty0 + 8 * slot, (round - 1) & 1, a.status, 501);
        if (!ok) break;
        const uint32_t dst = smem_u32(ring + (size_t)slot * kStage);
        const int nt = tiles_of(wk);
        mbar_expect_tx(full0 + 8 * slot, nt * kABytes + kBBytes);
        for (int t = 0; t < nt; ++t) bulk_load_1d(dst + t * kABytes, a_src(wk, t), kABytes, full0 + 8 * slot);
        bulk_load_1d(dst + TT * kABytes, b_src(wk), kBBytes, full0 + 8 * slot);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA
    // instruction descriptor: D f32, A e4m3, B e4m3, both K-major, N, M = 128
    const uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
    // A: K-adjacent core matrices (the 16-byte halves of a K step) 2048 B apart, row groups 128 B apart
    const uint64_t adesc_hi = ((uint64_t)(2048u >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
    // B: halves (N / 8) * 128 B apart, row groups 128 B apart
    const uint64_t bdesc_hi = ((uint64_t)(((N / 8) * 128u) >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
    int i = 0;
    for (int it = 0; wk.live(a) && ok; ++it) {
      const int b = it % ND;
      if (it >= ND) ok = mbar_wait(dfree0 + 8 * b, ((it - ND) / ND) & 1, a.status, 502);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      bool first = true;
      for (;; ++i) {
        const int slot = i % S;
        ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 503));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool last = wk.last_stage();
        const int nt = wk.tile * TT + TT <= a.ntiles ? TT : a.ntiles - wk.tile * TT;
        if (elect_one()) {
          const uint32_t abase = smem_u32(ring + (size_t)slot * kStage), bbase = abase + TT * kABytes;
#pragma unroll
          for (int t = 0; t < TT; ++t) {
            if (t < nt) {
#pragma unroll
              for (int st = 0; st < KS / 32; ++st) {
                const uint64_t adesc = adesc_hi | (uint64_t)(((abase + t * kABytes + st * 4096) >> 4) & 0x3FFF);
                const uint64_t bdesc = bdesc_hi | (uint64_t)(((bbase + st * (N * 32)) >> 4) & 0x3FFF);
                umma_f8_ss(tmem_base + b * (TT * N) + t * N, adesc, bdesc, idesc, (first && st == 0) ? 0u : 1u);
              }
            }
          }
          umma_commit(empty0 + 8 * slot);
          if (last) umma_commit(dfull0 + 8 * b);
        }
        __syncwarp();
        first = false;
        wk.next(a);
        if (last) {
          ++i;
          break;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q4 = warp & 3, hf = (warp - 2) >> 2;  // TMEM lane quarter (warp % 4), half of the rows
    const int r = q4 * 32 + lane;
    const int et = tid - 64;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    pdl_wait();  // the row scales of x come from the preparation kernel in front
    for (int it = 0; wk.live(a) && ok; ++it) {
      const int b = it % ND, group = wk.tile, split = wk.split;
      const int nt = group * TT + TT <= a.ntiles ? TT : a.ntiles - group * TT;
      // this role takes no part in the stages: on to the item's end
      wk.k = wk.k1 - 1;
      wk.next(a);
      // the rows' scales and biases are asked for before the wait, not behind it
      float scs[TT], bis[TT];
#pragma unroll
      for (int t = 0; t < TT; ++t) {
        const int row = (group * TT + t) * kTileRows + r;
        scs[t] = (t < nt && row < a.out_dim) ? __ldg(a.scale + row) : 0.f;
        bis[t] = (t < nt && a.bias && row < a.out_dim) ? __ldg(a.bias + row) : 0.f;
      }
      float xi[HM];  // 2^-e of this warp's activation rows
#pragma unroll
      for (int j = 0; j < HM; ++j) xi[j] = __ldg(a.xinv + hf * HM + j);
      ok = __all_sync(0xffffffffu, mbar_wait(dfull0 + 8 * b, (it / ND) & 1, a.status, 504));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float dot[TT][HM];
#pragma unroll
      for (int t = 0; t < TT; ++t) {
#pragma unroll
        for (int g = 0; g < HM / G; ++g) {
          float part[G];
#pragma unroll
          for (int j = 0; j < G; ++j) part[j] = 0.f;
          if (t < nt) {
#pragma unroll
            for (int p = P - 1; p >= 0; --p) {  // the smallest pieces first
              uint32_t v[G];
              tmem_ld_cols<G>(tmem_base + lane_base + b * (TT * N) + t * N + p * MP + hf * HM + g * G, v);
              tmem_ld_cols_wait<G>(v);
#pragma unroll
              for (int j = 0; j < G; ++j) part[j] = fmaf(__uint_as_float(v[j]), kPieceScale[p >> 1], part[j]);
            }
          }
#pragma unroll
          for (int j = 0; j < G; ++j) dot[t][g * G + j] = part[j];
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(dfree0 + 8 * b);
      if (a.cluster) {
        // The K splits of this group are the CTAs of this cluster (rank == split), one item each.
        // Ranks above 0 put their sums into rank 0's shared memory and arrive on its barrier (one
        // releasing arrival per warp); rank 0 waits, adds in split order — the order of the scratch
        // path, so the same bits — and stores.
        if (split != 0) {
#pragma unroll
          for (int t = 0; t < TT; ++t) {
            if (t < nt) {
#pragma unroll
              for (int j = 0; j < HM; ++j)
                cluster_store_f32(cluster_map(smem_u32(recv + ((size_t)((split - 1) * TT + t) * MP + hf * HM + j) * kTileRows + r), 0), dot[t][j]);
            }
          }
          __syncwarp();
          if (lane == 0) cluster_arrive_release(cluster_map(clbar, 0));
        } else {
          ok = __all_sync(0xffffffffu, mbar_wait_cluster(clbar, 0, a.status, 505));
          if (ok) {
#pragma unroll
            for (int t = 0; t < TT; ++t) {
              if (t < nt) {
                const int row = (group * TT + t) * kTileRows + r;
#pragma unroll
                for (int j = 0; j < HM; ++j) {
                  const int m = hf * HM + j;
                  float sum = dot[t][j];
                  for (int s2 = 1; s2 < a.splits; ++s2) sum += recv[((size_t)((s2 - 1) * TT + t) * MP + m) * kTileRows + r];
                  if (m < a.batch && row < a.out_dim) a.out[(size_t)m * a.out_dim + row] = fmaf(sum * xi[j], scs[t], bis[t]);
                }
              }
            }
          }
        }
        continue;
      }
#pragma unroll
      for (int t = 0; t < TT; ++t) {
        if (t >= nt) break;
        const int tile = group * TT + t;
        const int row = tile * kTileRows + r;
        const float sc = scs[t], bi = bis[t];
        if (a.splits == 1) {
#pragma unroll
          for (int j = 0; j < HM; ++j) {
            const int m = hf * HM + j;
            if (m < a.batch && row < a.out_dim) a.out[(size_t)m * a.out_dim + row] = fmaf(dot[t][j] * xi[j], sc, bi);
          }
        } else {
          // Partial sums of this K range go to scratch; the CTA that arrives last at the tile adds the
          // partials in split order (so the result does not depend on arrival order) and stores.
          float* part = a.scratch + ((size_t)tile * a.splits + split) * (MP * kTileRows);
#pragma unroll
          for (int j = 0; j < HM; ++j) part[(hf * HM + j) * kTileRows + r] = dot[t][j];
          __threadfence();
          asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
          if (et == 0) *last_flag = (atomicAdd(a.counters + tile, 1u) == (unsigned)a.splits - 1) ? 1 : 0;
          asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
          if (*last_flag) {
            __threadfence();
            const float* base = a.scratch + (size_t)tile * a.splits * (MP * kTileRows);
            float sum[HM];
#pragma unroll
            for (int j = 0; j < HM; ++j) sum[j] = 0.f;
            for (int s2 = 0; s2 < a.splits; ++s2) {  // a split's HM loads are independent: all in flight together
#pragma unroll
              for (int j = 0; j < HM; ++j) sum[j] += __ldcg(base + (size_t)s2 * (MP * kTileRows) + (hf * HM + j) * kTileRows + r);
            }
#pragma unroll
            for (int j = 0; j < HM; ++j) {
              const int m = hf * HM + j;
              if (m < a.batch && row < a.out_dim) a.out[(size_t)m * a.out_dim + row] = fmaf(sum[j] * xi[j], sc, bi);
            }
            if (et == 0) a.counters[tile] = 0;
          }
          asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        }
      }
    }
  }

  // ---- wind down: everyone meets, outstanding copies are drained, TMEM is returned ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0 && lane == 0 && *reinterpret_cast<volatile int*>(a.status) != 0) {
    // a waiter gave up: copies may still be in flight; give each ring slot a bounded chance to land
    for (int s = 0; s < S; ++s) {
      long long t0 = clock64();
      while (!mbar_try_wait(full0 + 8 * s, 0) && !mbar_try_wait(full0 + 8 * s, 1) && clock64() - t0 < kTimeoutCycles / 8) {
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kCols) : "memory");
  }
}

// ---- host side ----------------------------------------------------------------------------------

struct Fp8Bufs {
  unsigned char* xb = nullptr;
  float* xinv = nullptr;
  int* status = nullptr;
  float* scratch = nullptr;
  unsigned int* counters = nullptr;
};

// Per-device scratch, allocated on first use (or not at all when only its status is asked for);
// published only when every allocation and clearing has succeeded.
Fp8Bufs* fp8_bufs(int device, bool allocate = true) {
  static Fp8Bufs bufs[kMaxDevices];
  static bool ready[kMaxDevices] = {};
  static std::mutex mu;
  if (device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (ready[device]) return &bufs[device];
  if (!allocate) return nullptr;
  Fp8Bufs b;
  bool ok = cudaMalloc(&b.xb, kXbBytes) == cudaSuccess && cudaMalloc(&b.xinv, 64 * sizeof(float)) == cudaSuccess &&
            cudaMalloc(&b.status, 256) == cudaSuccess && cudaMalloc(&b.scratch, kScratchFloats * 4) == cudaSuccess &&
            cudaMalloc(&b.counters, kMaxCounters * 4) == cudaSuccess;
  ok = ok && cudaMemset(b.status, 0, 256) == cudaSuccess && cudaMemset(b.counters, 0, kMaxCounters * 4) == cudaSuccess &&
       cudaDeviceSynchronize() == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    cudaFree(b.xb);
    cudaFree(b.xinv);
    cudaFree(b.status);
    cudaFree(b.scratch);
    cudaFree(b.counters);
    return nullptr;
  }
  bufs[device] = b;
  ready[device] = true;
  return &bufs[device];
}

template <int N, int P, int MP, bool XBF16, int TT = 1>
int launch_pass(const goph_fp8_linear* w, float* out, const void* x, int nb, Fp8Bufs* bufs, cudaStream_t stream) {
  constexpr int KS = (N <= 64 && TT == 1) ? 256 : 128;
  constexpr int kStage = TT * kTileRows * KS + N * KS;
  DeviceState& st = device_state(w->device);
  Fp8Args a;
  memset(&a, 0, sizeof a);
  a.w = w->tiled;
  a.xb = bufs->xb;
  a.xinv = bufs->xinv;
  a.scale = w->scale;
  a.bias = w->bias;
  a.out = out;
  a.status = bufs->status;
  a.scratch = bufs->scratch;
  a.counters = bufs->counters;
  a.out_dim = w->out_dim;
  a.in_dim = w->in_dim;
  a.batch = nb;
  a.ntiles = (w->out_dim + kTileRows - 1) / kTileRows;
  a.nks = w->in_dim / KS;
  int max_items = (int)(kScratchFloats / ((size_t)MP * kTileRows));
  if (a.ntiles > (int)kMaxCounters) max_items = 0;
  const int ngroups = (a.ntiles + TT - 1) / TT;  // items are groups of TT row tiles x K splits
  a.splits = options().mlx_splits > 0 ? (options().mlx_splits < a.nks ? options().mlx_splits : a.nks)
                                      : tc_choose_splits(ngroups, a.nks, st.sm_count, max_items / TT, 2.f + TT * MP / 16.f);
  while (a.splits > 1 && (long)a.ntiles * a.splits > max_items) --a.splits;
  a.items = ngroups * a.splits;
  const int grid = a.items < st.sm_count ? a.items : st.sm_count;
  // K splits that all run at once, one item per CTA, whose partial sums fit the receive area: a cluster per group
  const bool want_cluster = options().mlx_cluster && a.splits > 1 && a.splits <= 8 && a.items == grid &&
                            (size_t)(a.splits - 1) * TT * MP * kTileRows * 4 <= (size_t)kRecvBytes;
  const size_t extra = 2048 + (want_cluster ? kRecvBytes : 0);
  int stages = (int)((kSmemBudget - extra) / kStage);
  if (stages > kMaxStages) stages = kMaxStages;
  a.stages = stages;
  size_t smem = (size_t)stages * kStage + extra;
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM (the kernel owns all of TMEM)

  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(MP, (w->in_dim + kPrepSlice - 1) / kPrepSlice);
  cfg.blockDim = dim3(256);
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, fp8_prep_x_kernel<P, XBF16>, x, bufs->xb, bufs->xinv, nb, w->in_dim, N, MP));
  auto kern = fp8_mma_kernel<N, P, MP, KS, TT>;
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
      if (!known[w->device][a.splits]) {
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
          cudaGetLastError();
          n = 0;
        }
        room[w->device][a.splits] = n;
        known[w->device][a.splits] = true;
      }
      resident = room[w->device][a.splits];
    }
    if (resident * a.splits >= grid) a.cluster = 1;
    else cfg.numAttrs = 1;
  }
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  return GOPH_OK;
}

// Row-major bytes -> blocks of K-major core matrices; one thread per 16-byte unit.  Flags the two NaN codes.
__global__ void fp8_tile_kernel(const unsigned char* __restrict__ w, unsigned char* __restrict__ tiled, int out_dim, int in_dim,
                                int ntiles, int nchunks, int* nan_flag) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t nblocks = (size_t)ntiles * nchunks;
  if (idx >= nblocks * (128 * 16)) return;
  size_t blk = idx / (128 * 16);
  int rem = (int)(idx - blk * (128 * 16));
  int tile = (int)(blk / nchunks), chunk = (int)(blk - (size_t)tile * nchunks);
  int r = rem >> 4, u = rem & 15, row = tile * 128 + r;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (row < out_dim) {
    v = *reinterpret_cast<const uint4*>(w + (size_t)row * in_dim + chunk * 256 + u * 16);
    const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
    bool nan = false;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t m = ws[k] & 0x7F7F7F7Fu;
      nan = nan || (m & 0xFFu) == 0x7Fu || (m & 0xFF00u) == 0x7F00u || (m & 0xFF0000u) == 0x7F0000u || (m >> 24) == 0x7Fu;
    }
    if (nan) *nan_flag = 1;
  }
  *reinterpret_cast<uint4*>(tiled + blk * kBlockBytes + (u >> 1) * 4096 + (u & 1) * 2048 + (r >> 3) * 128 + (r & 7) * 16) = v;
}

__global__ void fp8_dequant_tiled_kernel(const unsigned char* __restrict__ tiled, const float* __restrict__ scale,
                                         float* __restrict__ out, int out_dim, int in_dim, int nchunks) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)out_dim * in_dim) return;
  int row = (int)(i / in_dim), col = (int)(i - (size_t)row * in_dim);
  int chunk = col >> 8, k = col & 255, u = k >> 4, r = row & 127;
  const unsigned char* blk = tiled + ((size_t)(row >> 7) * nchunks + chunk) * kBlockBytes;
  unsigned char b = blk[(u >> 1) * 4096 + (u & 1) * 2048 + (r >> 3) * 128 + (r & 7) * 16 + (k & 15)];
  __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  out[i] = __fmul_rn(__half2float(*reinterpret_cast<__half*>(&hr)), scale[row]);
}

}  // namespace

// Passes of up to 32 activation rows.  f32 activations: six pieces (an f32 exactly); bf16 activations:
// two pieces.
int tc_gemm_fp8(const goph_fp8_linear* w, float* out, const void* x, bool x_bf16, int batch, cudaStream_t stream) {
  if (!w->tiled) return fail(GOPH_E_UNSUPPORTED, "FP8 linear is not in the tensor-core layout");
  if (w->in_dim % kChunkK != 0 || w->in_dim > kMaxIn)
    return fail(GOPH_E_UNSUPPORTED, "FP8 tensor-core path: in_dim=%d is not a multiple of 256 up to %d", w->in_dim, kMaxIn);
  if ((uintptr_t)x % 16) return fail(GOPH_E_INVALID, "x must be 16-byte aligned");
  Fp8Bufs* bufs = fp8_bufs(w->device);
  if (!bufs) return fail(GOPH_E_NOMEM, "cannot allocate the FP8 tensor-core path's device scratch");
  const size_t xstride = (size_t)w->in_dim * (x_bf16 ? 2 : 4);
  for (int b0 = 0; b0 < batch;) {
    const int left = batch - b0;
    const void* xp = static_cast<const unsigned char*>(x) + (size_t)b0 * xstride;
    float* op = out + (size_t)b0 * w->out_dim;
    int rc, nb;
    if (x_bf16) {
      // two pieces hold a bf16 value; from 17 rows two row tiles share each B tile
      if (options().fp8_convert && left > 32) return tc_gemm_fp8_converted(w, op, xp, true, left, stream);
      if (left <= 8) rc = launch_pass<16, 2, 8, true>(w, op, xp, nb = left, bufs, stream);
      else if (left <= 16) rc = launch_pass<32, 2, 16, true>(w, op, xp, nb = left, bufs, stream);
      else if (left <= 32) rc = launch_pass<64, 2, 32, true, 2>(w, op, xp, nb = left, bufs, stream);
      else rc = launch_pass<128, 2, 64, true, 2>(w, op, xp, nb = left < 64 ? left : 64, bufs, stream);
    } else {
      // six pieces hold an f32 exactly
      if (left <= 2) rc = launch_pass<16, 6, 2, false>(w, op, xp, nb = left, bufs, stream);
      else if (left <= 4) rc = launch_pass<32, 6, 4, false>(w, op, xp, nb = left, bufs, stream);
      else if (left <= 8) rc = launch_pass<48, 6, 8, false>(w, op, xp, nb = left, bufs, stream);
      else if (left <= 16) rc = launch_pass<96, 6, 16, false>(w, op, xp, nb = left, bufs, stream);
      else rc = launch_pass<192, 6, 32, false>(w, op, xp, nb = left < 32 ? left : 32, bufs, stream);
    }
    if (rc) return rc;
    b0 += nb;
  }
  return GOPH_OK;
}

bool tc_fp8_supported(int in_dim) { return in_dim % kChunkK == 0 && in_dim <= kMaxIn; }

int tc_fp8_make_tiled(goph_fp8_linear* w, int* has_nan) {
  const int ntiles = (w->out_dim + kTileRows - 1) / kTileRows, nchunks = w->in_dim / kChunkK;
  const size_t bytes = (size_t)ntiles * nchunks * kBlockBytes;
  unsigned char* t = nullptr;
  int* flag = nullptr;
  GOPH_CUDA(cudaMalloc(&t, bytes));
  cudaError_t e = cudaMalloc(&flag, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(flag, 0, sizeof(int));
  if (e == cudaSuccess) {
    size_t threads = (size_t)ntiles * nchunks * 128 * 16;
    fp8_tile_kernel<<<(unsigned)((threads + 255) / 256), 256>>>(w->weight, t, w->out_dim, w->in_dim, ntiles, nchunks, flag);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpy(has_nan, flag, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(flag);
  if (e != cudaSuccess) {
    cudaFree(t);
    return fail_cuda(e, "fp8_tile_kernel");
  }
  if (*has_nan) {
    cudaFree(t);
    return GOPH_OK;
  }
  w->tiled = t;
  return GOPH_OK;
}

int tc_fp8_dequant_tiled(const goph_fp8_linear* w, float* out, cudaStream_t stream) {
  size_t n = (size_t)w->out_dim * w->in_dim;
  fp8_dequant_tiled_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(w->tiled, w->scale, out, w->out_dim, w->in_dim,
                                                                            w->in_dim / kChunkK);
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

int fp8_mma_status(int device) {
  Fp8Bufs* b = fp8_bufs(device, false);
  if (!b) return 0;
  int v = 0;
  if (cudaMemcpy(&v, b->status, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return v;
}

void fp8_mma_status_clear(int device) {
  Fp8Bufs* b = fp8_bufs(device, false);
  if (b) cudaMemset(b->status, 0, sizeof(int));
}

}  // namespace goph
