// MLX 4-bit weights on the 5th-generation tensor cores (tcgen05 + TMEM), for any batch.
//
// Why a GEMV goes to the tensor pipe: at B200's 7.7 TB/s one SM has to consume ~47 nibbles
// per clock.  Turning a nibble into an f32 and multiplying it on the CUDA cores costs one
// logic op per nibble on the half-rate integer pipe plus the FMA, which caps a CUDA-core
// kernel well under the HBM roofline.  Here a logic op makes TWO bf16 operands, the products
// run on the tensor pipe, and the CUDA cores only apply the per-group scales.
//
// Arithmetic (exact up to f32 accumulation order):
//   * A operand: the nibble n is placed in the low mantissa bits of a bf16 with exponent 2^7,
//     which reads as the integer 128 + n — exact, no rounding.
//   * B operand: each activation row x (f32) is split into bf16 pieces hi + mid + lo = x
//     (exactly), one B row per piece; a caller that knows x holds bf16 values uses one piece.
//   * One accumulator block per 64-element group: D_g[row, col] = sum_{k in g} (128 + n) x.
//     The epilogue forms  s_g * (D_g - 128 * xsum_g) + b_g * xsum_g  in f32 and adds it to the
//     row's running sum, which is mlx.GemvTo's expression (backends/mlx/gemv.go:178-209).
//
// Pipeline of one CTA (persistent over 128-row tiles, 192 threads):
//   warp 4   TMA producer: one 2-D tensor-map copy (128 rows x 128 B, 128B swizzle) of packed
//            nibbles and one (128 rows x 16 B) of {scale,bias} pairs per 256-element K chunk
//            into a shared-memory ring guarded by full/empty mbarriers.
//   warps 0-3  thread r owns row r of the tile (TMEM lane r): reads its 128 bytes from the
//            swizzled stage, widens them to 128 bf16 pairs, tcgen05.st's them into the A
//            buffer in TMEM, writes its share of the B tile (x pieces) to shared memory, and
//            two stages later reads D back with tcgen05.ld for the scale epilogue.
//   warp 5   one thread issues 16 tcgen05.mma (M=128, N=16|32, K=16) per stage, A from TMEM,
//            B from shared memory, and commits to an mbarrier.
// Every wait is bounded: after ~2 s a waiter records a code in the status word and the CTA
// winds down (TMEM freed, outstanding copies drained) instead of spinning.
#include <cuda.h>
#include <string.h>

#include "goph_internal.cuh"
#include "mlx_mma.cuh"

namespace goph {

namespace {

constexpr int kTileRows = 128;
constexpr int kChunkK = 256;                  // elements per pipeline stage
constexpr int kStageWBytes = kTileRows * 128; // packed nibbles of a stage
constexpr int kStageMBytes = kTileRows * 16;  // {scale,bias} bf16 pairs, 4 groups of 64
constexpr int kStageBytes = kStageWBytes + kStageMBytes;
constexpr int kRowThreads = 128;
constexpr int kThreadsMMA = 192;
constexpr long long kTimeoutCycles = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait: false after ~2 s, with `code` left in the status word.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kTimeoutCycles) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Waits for the loads above; the registers are listed so no use of them can move before it.
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem descriptor]; issued by one thread.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// bf16 pieces of an f32 by truncation: x = hi + mid + lo exactly (8 significant bits each).
__device__ __forceinline__ void split3(float x, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  uint32_t h = __float_as_uint(x) & 0xFFFF0000u;
  float r1 = x - __uint_as_float(h);
  uint32_t m = __float_as_uint(r1) & 0xFFFF0000u;
  float r2 = r1 - __uint_as_float(m);
  hi = h >> 16;
  mid = m >> 16;
  lo = __float_as_uint(r2) >> 16;
}

}  // namespace

struct MmaArgs {
  const float* x;        // [batch][in_dim]
  float* out;            // [batch][out_dim]
  int* status;           // device word: 0 ok, otherwise the first wait that gave up
  float* scratch;        // split-K partial sums [item][batch][128]
  unsigned int* counters;  // per-tile arrival counters, zero between launches
  int out_dim, in_dim;
  int batch;             // activation rows of this launch (<= MB of the instantiation)
  int ntiles;            // ceil(out_dim / 128)
  int nchunks;           // in_dim / 256
  int splits;            // CTAs sharing the K range of one tile
  int items;             // ntiles * splits
  int stages;            // depth of the shared-memory ring
};

constexpr int kConvWarps = 8, kEpiWarps = 4;
constexpr int kConvThreads = kConvWarps * 32, kEpiThreads = kEpiWarps * 32;
constexpr int kWarpTMA = kConvWarps + kEpiWarps, kWarpMMA = kWarpTMA + 1;
constexpr int kThreadsV2 = (kWarpMMA + 1) * 32;

// Shared-memory plan (dynamic, 1024-byte aligned base): ring of stages (weights then meta),
// 2 B tiles (16 K-steps x N rows x 32 B), the xsum table, mbarriers, the TMEM base holder.
template <int N>
struct MmaSmem {
  static constexpr int kBTileBytes = 16 * N * 32;
  static __host__ __device__ size_t bytes(int stages, int batch, int in_dim) {
    return (size_t)stages * kStageBytes + 2 * kBTileBytes + (size_t)batch * (in_dim / 64) * 4 + 1024 + 512;
  }
};

// Walks the (tile, chunk) stages of this CTA's work items in the order every role uses.
struct StageWalk {
  int w, tile, split, c, c1;
  __device__ __forceinline__ void open(const MmaArgs& a) {
    tile = w / a.splits;
    split = w - tile * a.splits;
    c = split * a.nchunks / a.splits;
    c1 = (split + 1) * a.nchunks / a.splits;
  }
  __device__ __forceinline__ StageWalk(const MmaArgs& a) : w(blockIdx.x) {
    if (w < a.items) open(a);
  }
  __device__ __forceinline__ bool live(const MmaArgs& a) const { return w < a.items; }
  __device__ __forceinline__ bool last_chunk() const { return c + 1 == c1; }
  __device__ __forceinline__ void next(const MmaArgs& a) {
    if (++c == c1) {
      w += gridDim.x;
      if (w < a.items) open(a);
    }
  }
};

template <int N, int PIECES, int MB>
__global__ void __launch_bounds__(kThreadsV2, 1)
mlx_mma_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap mmap,
               const __grid_constant__ MmaArgs a) {
  static_assert(MB * PIECES <= N, "activation pieces must fit the N columns");
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  constexpr int kBTile = MmaSmem<N>::kBTileBytes;
  const int S = a.stages;
  unsigned char* ring = smem;
  unsigned char* btile = ring + (size_t)S * kStageBytes;       // 2 tiles
  float* xsum = reinterpret_cast<float*>(btile + 2 * kBTile);  // [batch][groups]
  const int groups = a.in_dim / 64;
  uint64_t* bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(xsum + (size_t)a.batch * groups) + 15) & ~uintptr_t(15));
  // bars: full[S], empty[S], a_ready[2], mma_done[2], d_free[2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 6);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + S);
  const uint32_t aready0 = smem_u32(bars + 2 * S), mdone0 = smem_u32(bars + 2 * S + 2), dfree0 = smem_u32(bars + 2 * S + 4);

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kConvThreads + kEpiThreads);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(aready0 + 8 * b, kConvThreads);
      mbar_init(mdone0 + 8 * b, 1);
      mbar_init(dfree0 + 8 * b, kEpiThreads);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kWarpMMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // zero the B tiles once: rows no activation piece maps to stay zero for the whole launch
  for (int i = tid; i < 2 * kBTile / 16; i += kThreadsV2) reinterpret_cast<uint4*>(btile)[i] = make_uint4(0, 0, 0, 0);
  // per-group sums of x
  for (int i = tid; i < a.batch * groups; i += kThreadsV2) {
    const float* p = a.x + (size_t)(i / groups) * a.in_dim + (size_t)(i % groups) * 64;
    float s = 0.f;
    for (int k = 0; k < 64; k += 4) {
      float4 v = __ldg(reinterpret_cast<const float4*>(p + k));
      s += (v.x + v.y) + (v.z + v.w);
    }
    xsum[i] = s;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmemA0 = tmem_base, tmemD0 = tmem_base + 256;  // A: 2 x 128 cols; D: 2 x 4N cols
  bool ok = true;
  StageWalk sw(a);

  if (warp == kWarpTMA) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; sw.live(a) && ok; ++i, sw.next(a)) {
        int slot = i % S, round = i / S;
        if (round > 0) ok = mbar_wait(empty0 + 8 * slot, (round - 1) & 1, a.status, 1);
        if (!ok) break;
        uint32_t dst = smem_u32(ring + (size_t)slot * kStageBytes);
        mbar_expect_tx(full0 + 8 * slot, kStageBytes);
        tma_load_2d(dst, &wmap, sw.c * 128, sw.tile * kTileRows, full0 + 8 * slot);
        tma_load_2d(dst + kStageWBytes, &mmap, sw.c * 16, sw.tile * kTileRows, full0 + 8 * slot);
      }
    }
  } else if (warp == kWarpMMA) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: D f32, A bf16, B bf16, both K-major, N, M=128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
      constexpr uint32_t kLBO = (N / 8) * 128, kSBO = 128;  // K-adjacent / N-adjacent core matrices
      for (int i = 0; sw.live(a) && ok; ++i, sw.next(a)) {
        int b = i & 1;
        ok = mbar_wait(aready0 + 8 * b, (i >> 1) & 1, a.status, 2);
        if (ok && i >= 2) ok = mbar_wait(dfree0 + 8 * b, ((i - 2) >> 1) & 1, a.status, 5);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t bbase = smem_u32(btile + (size_t)b * kBTile);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            int step = g * 4 + j;
            uint64_t desc = (uint64_t)(((bbase + step * (N * 32)) >> 4) & 0x3FFF) | ((uint64_t)(kLBO >> 4) << 16) |
                            ((uint64_t)(kSBO >> 4) << 32) | (1ull << 46);
            umma_ts(tmemD0 + b * (4 * N) + g * N, tmemA0 + b * 128 + step * 8, desc, idesc, j > 0 ? 1u : 0u);
          }
        }
        umma_commit(mdone0 + 8 * b);
      }
    }
  } else if (warp < kConvWarps) {
    // ------------------------------------------------------------------ converters
    // Thread = (row r of the tile, half h of the stage's eight 16-byte units).
    const int q = warp & 3, h = warp >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    // B-tile share of the h == 0 threads: K-step j, half kc, pair p (elements k and k+4).
    const int bj = r >> 3, bkc = (r >> 2) & 1, bp = r & 3;
    float xn0[MB], xn1[MB];
    auto fetch_x = [&](int chunk) {
      int k = chunk * kChunkK + bj * 16 + bkc * 8 + bp;
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        bool in = m < a.batch;
        xn0[m] = in ? __ldg(a.x + (size_t)m * a.in_dim + k) : 0.f;
        xn1[m] = in ? __ldg(a.x + (size_t)m * a.in_dim + k + 4) : 0.f;
      }
    };
    if (h == 0 && sw.live(a)) fetch_x(sw.c);
    for (int i = 0; sw.live(a) && ok; ++i) {
      int b = i & 1, slot = i % S;
      if (i >= 2) ok = __all_sync(0xffffffffu, mbar_wait(mdone0 + 8 * b, ((i - 2) >> 1) & 1, a.status, 3));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 4));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned char* st = ring + (size_t)slot * kStageBytes;
      // ---- widen this row's half of the stage (128 nibbles) into the A buffer ----
      uint4 qv[4];
#pragma unroll
      for (int uu = 0; uu < 4; ++uu) {
        int u = h * 4 + uu;
        qv[uu] = *reinterpret_cast<const uint4*>(st + r * 128 + ((u ^ (r & 7)) << 4));
      }
#pragma unroll
      for (int uu = 0; uu < 4; ++uu) {
        uint32_t ws[4] = {qv[uu].x, qv[uu].y, qv[uu].z, qv[uu].w};
        uint32_t regs[16];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          // nibble -> top mantissa bits of a bf16 under 2^4: the integer 16 + n, exactly
          constexpr uint32_t MK = 0x00780078u, EX = 0x41804180u;
          regs[4 * w + 0] = ((ws[w] << 3) & MK) | EX;  // elements (0,4) of the word
          regs[4 * w + 1] = ((ws[w] >> 1) & MK) | EX;  // (1,5)
          regs[4 * w + 2] = ((ws[w] >> 5) & MK) | EX;  // (2,6)
          regs[4 * w + 3] = ((ws[w] >> 9) & MK) | EX;  // (3,7)
        }
        tmem_st16(tmemA0 + lane_base + b * 128 + (h * 4 + uu) * 16, regs);
      }
      // ---- the B tile of this stage (x pieces), then prefetch the next stage's x ----
      if (h == 0) {
        unsigned char* bt = btile + (size_t)b * kBTile + bj * (N * 32) + bkc * ((N / 8) * 128) + bp * 4;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          if (PIECES == 3) {
            uint32_t h0, m0, l0, h1, m1, l1;
            split3(xn0[m], h0, m0, l0);
            split3(xn1[m], h1, m1, l1);
            constexpr int dummy = 0;
            (void)dummy;
            int n = 3 * m;
            *reinterpret_cast<uint32_t*>(bt + (n >> 3) * 128 + (n & 7) * 16) = h0 | (h1 << 16);
            *reinterpret_cast<uint32_t*>(bt + ((n + 1) >> 3) * 128 + ((n + 1) & 7) * 16) = m0 | (m1 << 16);
            *reinterpret_cast<uint32_t*>(bt + ((n + 2) >> 3) * 128 + ((n + 2) & 7) * 16) = l0 | (l1 << 16);
          } else {
            *reinterpret_cast<uint32_t*>(bt + (m >> 3) * 128 + (m & 7) * 16) =
                (__float_as_uint(xn0[m]) >> 16) | (__float_as_uint(xn1[m]) & 0xFFFF0000u);
          }
        }
      }
      sw.next(a);
      if (h == 0 && sw.live(a)) fetch_x(sw.c);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(aready0 + 8 * b);
      mbar_arrive(empty0 + 8 * slot);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int r = q * 32 + lane;  // row of the tile == TMEM lane
    const int et = tid - kConvThreads;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    float acc[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = 0.f;
    for (int i = 0; sw.live(a) && ok; ++i) {
      int b = i & 1, slot = i % S;
      ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * slot, (i / S) & 1, a.status, 6));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(mdone0 + 8 * b, (i >> 1) & 1, a.status, 7));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint4 mv = *reinterpret_cast<const uint4*>(ring + (size_t)slot * kStageBytes + kStageWBytes + r * 16);
      const uint32_t meta[4] = {mv.x, mv.y, mv.z, mv.w};
      uint32_t t[4][16];
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ld16(tmemD0 + lane_base + b * (4 * N) + g * N, t[g]);
      tmem_wait_ld(t[0]);
      tmem_wait_ld(t[1]);
      tmem_wait_ld(t[2]);
      tmem_wait_ld(t[3]);
      uint32_t t2[4][16];
      if (N == 32 && MB * PIECES > 16) {
#pragma unroll
        for (int g = 0; g < 4; ++g) tmem_ld16(tmemD0 + lane_base + b * (4 * N) + g * N + 16, t2[g]);
        tmem_wait_ld(t2[0]);
        tmem_wait_ld(t2[1]);
        tmem_wait_ld(t2[2]);
        tmem_wait_ld(t2[3]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(dfree0 + 8 * b);
      mbar_arrive(empty0 + 8 * slot);
      const float* xs_c = xsum + sw.c * 4;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float sc = __uint_as_float(meta[g] << 16), bi = __uint_as_float(meta[g] & 0xFFFF0000u);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          float xs = xs_c[m * groups + g];
          float dot;
          if (PIECES == 3) {
            auto col = [&](int cidx) { return __uint_as_float(cidx < 16 ? t[g][cidx & 15] : t2[g][cidx & 15]); };
            dot = (col(3 * m) + col(3 * m + 1)) + col(3 * m + 2);
          } else {
            dot = __uint_as_float(m < 16 ? t[g][m & 15] : t2[g][m & 15]);
          }
          acc[m] = fmaf(sc, dot - 16.f * xs, acc[m]);
          acc[m] = fmaf(bi, xs, acc[m]);
        }
      }
      const bool item_done = sw.last_chunk();
      const int tile = sw.tile, split = sw.split;
      sw.next(a);
      if (!item_done) continue;
      const int row = tile * kTileRows + r;
      if (a.splits == 1) {
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          if (m < a.batch && row < a.out_dim) a.out[(size_t)m * a.out_dim + row] = acc[m];
          acc[m] = 0.f;
        }
      } else {
        // Partial sums of this K range go to scratch; the CTA that arrives last at the tile adds
        // the partials in split order (so the result does not depend on arrival order) and stores.
        float* part = a.scratch + ((size_t)tile * a.splits + split) * (MB * kTileRows);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          part[m * kTileRows + r] = acc[m];
          acc[m] = 0.f;
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (et == 0) *last_flag = (atomicAdd(a.counters + tile, 1u) == (unsigned)a.splits - 1) ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (*last_flag) {
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- host side --------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

bool mlx_mma_supported(const goph_mlx_weight* w) {
  return w->sb_bf16 && w->group_size == 64 && w->in_dim % kChunkK == 0 && ((uintptr_t)w->qweight % 16) == 0 &&
         ((uintptr_t)w->sb % 16) == 0;
}

int mlx_mma_make_maps(goph_mlx_weight* w) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(GOPH_E_UNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap* maps = new CUtensorMap[2];
  cuuint64_t dims[2] = {(cuuint64_t)w->in_dim / 2, (cuuint64_t)w->out_dim};
  cuuint64_t strides[1] = {(cuuint64_t)w->in_dim / 2};
  cuuint32_t box[2] = {128, (cuuint32_t)kTileRows}, elem[2] = {1, 1};
  CUresult r = enc(&maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w->qweight, dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    cuuint64_t mdims[2] = {(cuuint64_t)w->groups * 4, (cuuint64_t)w->out_dim};
    cuuint64_t mstrides[1] = {(cuuint64_t)w->groups * 4};
    cuuint32_t mbox[2] = {16, (cuuint32_t)kTileRows};
    r = enc(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w->sb, mdims, mstrides, mbox, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    delete[] maps;
    return fail(GOPH_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  }
  w->tmaps = maps;
  return GOPH_OK;
}

void mlx_mma_free_maps(goph_mlx_weight* w) {
  delete[] reinterpret_cast<CUtensorMap*>(w->tmaps);
  w->tmaps = nullptr;
}

struct MmaDeviceBufs {
  int* status = nullptr;
  float* scratch = nullptr;
  unsigned int* counters = nullptr;
};
// Fixed-size device scratch of the split-K fix-up: at most 2 x SM-count items of 128 rows x 32
// activation rows, plus one counter per tile.  Allocated once per device.
constexpr size_t kScratchFloats = (size_t)2 * 160 * kTileRows * 32;
constexpr size_t kMaxCounters = 4096;

static MmaDeviceBufs* device_bufs(int device) {
  static MmaDeviceBufs bufs[kMaxDevices];
  MmaDeviceBufs& b = bufs[device];
  if (!b.status) {
    if (cudaMalloc(&b.status, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMalloc(&b.scratch, kScratchFloats * sizeof(float)) != cudaSuccess) return nullptr;
    if (cudaMalloc(&b.counters, kMaxCounters * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cudaMemset(b.status, 0, sizeof(int));
    cudaMemset(b.counters, 0, kMaxCounters * sizeof(unsigned int));
    cudaDeviceSynchronize();
  }
  return &b;
}

int mlx_mma_status(int device) {
  MmaDeviceBufs* b = device_bufs(device);
  int v = -1;
  if (b) cudaMemcpy(&v, b->status, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

template <int N, int PIECES, int MB>
static int launch_one(const goph_mlx_weight* w, const MmaArgs& a0, cudaStream_t stream) {
  MmaArgs a = a0;
  DeviceState& st = device_state(w->device);
  size_t fixed = MmaSmem<N>::bytes(0, a.batch, a.in_dim);
  int stages = (int)(((size_t)kSmemBudget - fixed) / kStageBytes);
  if (stages > 8) stages = 8;
  if (stages < 3)
    return fail(GOPH_E_UNSUPPORTED, "tensor-core path: activations of %d x %d leave no room for the ring", a.batch, a.in_dim);
  a.stages = stages;
  // K split: enough (tile, split) items to occupy the SMs, bounded by the chunks and the scratch
  int splits = 1;
  if (a.ntiles < st.sm_count) {
    splits = st.sm_count / a.ntiles;
    if (splits > a.nchunks) splits = a.nchunks;
    if (splits < 1) splits = 1;
    while (splits > 1 && ((size_t)a.ntiles * splits * kTileRows * MB > kScratchFloats || (size_t)a.ntiles > kMaxCounters)) --splits;
  }
  if (options().mlx_splits > 0) splits = options().mlx_splits < a.nchunks ? options().mlx_splits : a.nchunks;
  a.splits = splits;
  a.items = a.ntiles * splits;
  size_t smem = MmaSmem<N>::bytes(stages, a.batch, a.in_dim);
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: each allocates all 512 TMEM columns
  auto kern = mlx_mma_kernel<N, PIECES, MB>;
  GOPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = a.items < st.sm_count ? a.items : st.sm_count;
  const CUtensorMap* maps = reinterpret_cast<const CUtensorMap*>(w->tmaps);
  kern<<<grid, kThreadsV2, smem, stream>>>(maps[0], maps[1], a);
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

int mlx_mma_launch(const goph_mlx_weight* w, float* out, const float* x, int batch, int pieces, cudaStream_t stream) {
  if (!w->tmaps) return fail(GOPH_E_UNSUPPORTED, "weight has no tensor maps");
  MmaDeviceBufs* bufs = device_bufs(w->device);
  if (!bufs) return fail(GOPH_E_NOMEM, "cannot allocate the tensor-core path's device scratch");
  MmaArgs a;
  memset(&a, 0, sizeof a);
  a.status = bufs->status;
  a.scratch = bufs->scratch;
  a.counters = bufs->counters;
  a.out_dim = w->out_dim;
  a.in_dim = w->in_dim;
  a.ntiles = (w->out_dim + kTileRows - 1) / kTileRows;
  a.nchunks = w->in_dim / kChunkK;
  const int cap = pieces == 3 ? 10 : 32;  // activation rows one launch can take
  for (int b0 = 0; b0 < batch;) {
    int nb = batch - b0 < cap ? batch - b0 : cap;
    a.x = x + (size_t)b0 * w->in_dim;
    a.out = out + (size_t)b0 * w->out_dim;
    a.batch = nb;
    int rc;
    if (pieces == 3) {
      rc = nb == 1 ? launch_one<16, 3, 1>(w, a, stream)
         : nb == 2 ? launch_one<16, 3, 2>(w, a, stream)
         : nb <= 5 ? launch_one<16, 3, 5>(w, a, stream)
                   : launch_one<32, 3, 10>(w, a, stream);
    } else {
      rc = nb == 1 ? launch_one<16, 1, 1>(w, a, stream)
         : nb <= 4 ? launch_one<16, 1, 4>(w, a, stream)
         : nb <= 16 ? launch_one<16, 1, 16>(w, a, stream)
                    : launch_one<32, 1, 32>(w, a, stream);
    }
    if (rc) return rc;
    b0 += nb;
  }
  return GOPH_OK;
}

}  // namespace goph
