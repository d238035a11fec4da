// MLX 4-bit affine weights: upload, bit-exact dequantisation, and the dequant-fused
// GEMV / small-batch product.
//
// Replaces the reference's mlx_gemv / mlx_gemm / mlx_correct / gemv_q4sym PTX
// (backends/nvidia/ptx/mlx/mlx.go, ptx/q4/gemv.go) behind nvidia.GemvMLX,
// GemvMLXDirect and GemmMLX (backends/nvidia/runtime/mlx.go:287-488).  The arithmetic
// specification is mlx.GemvTo (backends/mlx/gemv.go:164-209):
//     out[r] = sum_g ( scale[r,g] * sum_{e in g} nibble*x  +  bias[r,g] * sum_{e in g} x ).
//
// Streaming kernel (mlx_gemv_kernel)
//   * A warp owns R consecutive rows at a time.  Lane l of iteration `it` owns the 16
//     bytes (32 nibbles, half of a 64-group) at unit u = 32*it + l of each of those rows,
//     so one warp instruction is a 512-byte coalesced, L1-bypassing load per row.
//   * x lives in shared memory as f32, permuted so that the eight float4 a lane needs
//     for its unit are read with conflict-free LDS.128 ([batch][it][slot][lane]).
//     Beside it sit two numbers per unit, c1 and c2 (below).
//   * A nibble n becomes an f32 by bit placement only: put it in the top mantissa bits
//     under a fixed exponent and the word reads as (K + n) for a constant K (16, or 256
//     for the partner nibble when one shift serves two nibbles).  The constant is
//     removed algebraically per unit:  sum (K+n)x = F,  sum n x = F - c1  with
//     c1 = sum K x precomputed once per unit; c2 = sum x feeds the bias term.
//   * Products are accumulated with fma.rn.f32x2 (two f32 FMAs per issue slot), one
//     f32 accumulator per (row, batch) pair, reduced across the warp by shuffles.
//   * The next step's weights are already in flight while the current step computes.
#include <stdlib.h>
#include <string.h>

#include <type_traits>
#include <vector>

#include "goph_internal.cuh"
#include "mlx_mma.cuh"
#include "tc_gemm.cuh"

namespace goph {

enum { UNPACK_EXACT = 0, UNPACK_PAIR = 1, UNPACK_CVT = 2 };

// Turns the eight nibbles of `w` into f[j] = off(j) + nibble_j.
template <int MODE>
struct Unpack;

// Every nibble is moved to mantissa bits 19..22 under exponent 2^4: f = 16 + n.
template <>
struct Unpack<UNPACK_EXACT> {
  static constexpr float kOffEven = 16.f, kOffOdd = 16.f;
  static __device__ __forceinline__ void run(uint32_t w, float (&f)[8]) {
    constexpr uint32_t M = 0x00780000u, E = 0x41800000u;
    f[0] = __uint_as_float(((w << 19) & M) | E);
    f[1] = __uint_as_float(((w << 15) & M) | E);
    f[2] = __uint_as_float(((w << 11) & M) | E);
    f[3] = __uint_as_float(((w << 7) & M) | E);
    f[4] = __uint_as_float(((w << 3) & M) | E);
    f[5] = __uint_as_float(((w >> 1) & M) | E);
    f[6] = __uint_as_float(((w >> 5) & M) | E);
    f[7] = __uint_as_float(((w >> 9) & M) | E);
  }
};

// One shift serves two neighbouring nibbles: the odd one lands on bits 19..22 under 2^4
// (16 + n), the even one on bits 15..18 under 2^8 (256 + n).
template <>
struct Unpack<UNPACK_PAIR> {
  static constexpr float kOffEven = 256.f, kOffOdd = 16.f;
  static __device__ __forceinline__ void run(uint32_t w, float (&f)[8]) {
    constexpr uint32_t MA = 0x00780000u, EA = 0x41800000u, MB = 0x00078000u, EB = 0x43800000u;
    uint32_t t0 = w << 15, t1 = w << 7, t2 = w >> 1, t3 = w >> 9;
    f[0] = __uint_as_float((t0 & MB) | EB);
    f[1] = __uint_as_float((t0 & MA) | EA);
    f[2] = __uint_as_float((t1 & MB) | EB);
    f[3] = __uint_as_float((t1 & MA) | EA);
    f[4] = __uint_as_float((t2 & MB) | EB);
    f[5] = __uint_as_float((t2 & MA) | EA);
    f[6] = __uint_as_float((t3 & MB) | EB);
    f[7] = __uint_as_float((t3 & MA) | EA);
  }
};

// Plain integer-to-float conversion of each nibble (no offset to remove).
template <>
struct Unpack<UNPACK_CVT> {
  static constexpr float kOffEven = 0.f, kOffOdd = 0.f;
  static __device__ __forceinline__ void run(uint32_t w, float (&f)[8]) {
    uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
    f[0] = (float)(lo & 0xFF);
    f[1] = (float)(hi & 0xFF);
    f[2] = (float)((lo >> 8) & 0xFF);
    f[3] = (float)((hi >> 8) & 0xFF);
    f[4] = (float)((lo >> 16) & 0xFF);
    f[5] = (float)((hi >> 16) & 0xFF);
    f[6] = (float)(lo >> 24);
    f[7] = (float)(hi >> 24);
  }
};

constexpr int kMaxSeg = 8;
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

struct MlxSeg {
  const uint4* w;   // packed rows, `units` uint4 per row
  const void* sb;   // {scale,bias} per (row, group)
  float* out;       // [batch][rows]
  int rows;
  int task0;        // index of this segment's first warp task
};

struct MlxArgs {
  MlxSeg seg[kMaxSeg];
  int nseg;
  int tasks;        // total warp tasks (row groups of R rows) over all segments
  const float* x;   // [batch][in_dim]
  int batch;
  int in_dim;
  int units;        // in_dim / 32
  int iters;        // ceil(units / 32)
  int groups;       // in_dim / group_size
  int ug_shift;     // log2(group_size / 32)
  int x_aligned;    // x is 16-byte aligned
  // Operation applied to x while it is staged (batch 1, 16-byte aligned vectors):
  //   1  v = x (+ pre_b); CTA 0 stores v to pre_hidden (which must not alias x or pre_b);
  //      staged x = (v * inv) * pre_w, inv = 1/sqrt(sum(v^2)/n + pre_eps)  — residual add + RMSNorm
  //   2  staged x = silu(x) * pre_b                                          — SiLU(gate) * up
  int pre_op;
  const float* pre_b;
  const float* pre_w;
  float* pre_hidden;
  float pre_eps;
};

// c1 = sum over a unit of (offset * x), c2 = sum of x, from the sums over the unit's even and odd
// elements; one definition so that every kernel rounds alike.
template <int MODE>
__device__ __forceinline__ float2 mlx_unit_consts(float se, float so) {
  return make_float2(__fmaf_rn(Unpack<MODE>::kOffEven, se, __fmul_rn(Unpack<MODE>::kOffOdd, so)), __fadd_rn(se, so));
}

// Shared memory: float4 xs[M][iters][8][32]; float2 xc[M][iters][32].
__host__ __device__ inline size_t mlx_smem_bytes(int M, int iters) {
  return (size_t)M * iters * (8 * 32 * 16 + 32 * 8);
}

template <int M, int MODE>
__device__ __forceinline__ void mlx_stage_x(const MlxArgs& a, float4* xs, float2* xc) {
  // Consecutive threads read consecutive 16 bytes of x (a warp asks the L2 for four lines, not for a
  // piece of thirty-two): float4 number t + 256*i of row m holds slot t%8 of unit (t + 256*i)/8 and goes
  // to xs[((m*iters + unit/32)*8 + slot)*32 + unit%32].  Four loads are in flight before the first store.
  const int n = M * a.iters;
  const int slot = threadIdx.x & 7, u0 = threadIdx.x >> 3;  // unit = it*32 + u0
  for (int j0 = 0; j0 < n; j0 += 4) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < n) {
        const int m = M == 1 ? 0 : j / a.iters, it = j - m * a.iters, unit = it * 32 + u0;
        if (m < a.batch && unit < a.units) {
          // plain (coherent) loads: inside a product list x may have been written earlier in this launch
          const float* p = a.x + (size_t)m * a.in_dim + (size_t)unit * 32 + slot * 4;
          if (a.x_aligned) {
            v[u] = *reinterpret_cast<const float4*>(p);
          } else {
            v[u] = make_float4(p[0], p[1], p[2], p[3]);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u < n) xs[((j0 + u) * 8 + slot) * 32 + u0] = v[u];
  }
  __syncthreads();
  const int nsum = M * a.iters * 32;
  for (int idx = threadIdx.x; idx < nsum; idx += kThreads) {
    int mi = idx >> 5, l = idx & 31;  // mi = m*iters + it
    float se = 0.f, so = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      float4 v = xs[(mi * 8 + s) * 32 + l];
      se += v.x + v.z;
      so += v.y + v.w;
    }
    xc[idx] = mlx_unit_consts<MODE>(se, so);
  }
  __syncthreads();
}

// Staging with the operation a.pre_op in front (see MlxArgs); batch 1.
template <int MODE>
__device__ __forceinline__ void mlx_stage_x_pre(const MlxArgs& a, float4* xs, float2* xc, int cta) {
  __shared__ float red[kWarps];
  const int total = a.iters * 256;
  float ss = 0.f;
  // consecutive threads take consecutive 16 bytes of the vectors (see mlx_stage_x); xs keeps its layout
  auto at = [](int idx) { return (((idx >> 8) * 8 + (idx & 7)) * 32) + ((idx >> 3) & 31); };
  for (int idx = threadIdx.x; idx < total; idx += kThreads) {
    const int slot = idx & 7, unit = idx >> 3;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (unit < a.units) {
      const size_t e0 = (size_t)unit * 32 + slot * 4;
      v = *reinterpret_cast<const float4*>(a.x + e0);
      if (a.pre_op == 1) {
        if (a.pre_b) {
          const float4 b = *reinterpret_cast<const float4*>(a.pre_b + e0);
          v = make_float4(__fadd_rn(v.x, b.x), __fadd_rn(v.y, b.y), __fadd_rn(v.z, b.z), __fadd_rn(v.w, b.w));
        }
        if (a.pre_hidden && cta == 0) *reinterpret_cast<float4*>(a.pre_hidden + e0) = v;
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
      } else {
        // single-precision exp (2 ulp) where the reference rounds an f64 exp to f32: every CTA
        // repeats this for the whole vector and the FP64 pipe of this part is slow
        const float4 u = *reinterpret_cast<const float4*>(a.pre_b + e0);
        v.x = __fmul_rn(__fdiv_rn(v.x, __fadd_rn(1.f, expf(-v.x))), u.x);
        v.y = __fmul_rn(__fdiv_rn(v.y, __fadd_rn(1.f, expf(-v.y))), u.y);
        v.z = __fmul_rn(__fdiv_rn(v.z, __fadd_rn(1.f, expf(-v.z))), u.z);
        v.w = __fmul_rn(__fdiv_rn(v.w, __fadd_rn(1.f, expf(-v.w))), u.w);
      }
    }
    xs[at(idx)] = v;
  }
  if (a.pre_op == 1) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) t += red[w];
    const float inv = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)a.in_dim), a.pre_eps)));
    for (int idx = threadIdx.x; idx < total; idx += kThreads) {
      const int slot = idx & 7, unit = idx >> 3;
      if (unit < a.units) {
        const float4 w = *reinterpret_cast<const float4*>(a.pre_w + (size_t)unit * 32 + slot * 4);
        float4 v = xs[at(idx)];
        v = make_float4(__fmul_rn(__fmul_rn(v.x, inv), w.x), __fmul_rn(__fmul_rn(v.y, inv), w.y),
                        __fmul_rn(__fmul_rn(v.z, inv), w.z), __fmul_rn(__fmul_rn(v.w, inv), w.w));
        xs[at(idx)] = v;
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < a.iters * 32; idx += kThreads) {
    const int mi = idx >> 5, l = idx & 31;
    float se = 0.f, so = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      float4 v = xs[(mi * 8 + s) * 32 + l];
      se += v.x + v.z;
      so += v.y + v.w;
    }
    xc[idx] = mlx_unit_consts<MODE>(se, so);
  }
  __syncthreads();
}

// The streaming product for one launch's worth of work, as CTA `cta` of `nctas`.  `wait` runs on
// every thread after the first weight loads are issued and before x is read: it is where the
// producer of x is waited for.
template <int R, int M, int MODE, bool SB_BF16, class Wait>
__device__ __forceinline__ void mlx_gemv_body(const MlxArgs& a, unsigned char* smem_raw, int cta, int nctas, Wait wait) {
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)M * a.iters * 8 * 32 * 16);

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int task_stride = nctas * kWarps;
  const int iters = a.iters;
  const int units = a.units;
  typedef typename std::conditional<SB_BF16, uint32_t, float2>::type SbT;

  // Per-task state: where this warp's R rows start (16-byte units / table entries) and where
  // their results go.  Computed once per task, not per iteration.
  struct Rows {
    const uint4* w[R];
    const SbT* sb[R];
    float* out;
    int rows, row0;
  };
  auto open_task = [&](int task, Rows& t) {
    int seg = 0;
#pragma unroll
    for (int s = 1; s < kMaxSeg; ++s)
      if (s < a.nseg && task >= a.seg[s].task0) seg = s;
    const MlxSeg& sg = a.seg[seg];
    t.row0 = (task - sg.task0) * R;
    t.rows = sg.rows;
    t.out = sg.out;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int row = t.row0 + r < sg.rows ? t.row0 + r : sg.rows - 1;
      t.w[r] = sg.w + (size_t)row * units;
      t.sb[r] = reinterpret_cast<const SbT*>(sg.sb) + (size_t)row * a.groups;
    }
  };
  struct Tile {
    uint4 w[R];
    SbT sb[R];  // as loaded: nothing is computed from a tile before its step, so a load never blocks the issue of the next
  };
  auto load_tile = [&](const Rows& t, int it, Tile& d) {
    int unit = it * 32 + lane;
    if (unit >= units) unit = units - 1;  // x is zero there; any finite weight will do
    const int grp = unit >> a.ug_shift;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      d.w[r] = ld_stream(t.w[r] + unit);
      d.sb[r] = __ldg(t.sb[r] + grp);
    }
  };
  auto tile_scale = [](const SbT& v) -> float {
    if constexpr (SB_BF16) return __uint_as_float(v << 16);
    else return v.x;
  };
  auto tile_bias = [](const SbT& v) -> float {
    if constexpr (SB_BF16) return __uint_as_float(v & 0xFFFF0000u);
    else return v.y;
  };

  // A warp's work is a sequence of steps (task, iteration); the tiles of the next D steps are in
  // flight in a ring of registers.  The weights do not depend on the producer of x: the ring is
  // filled first, then the producer is waited for and x is staged.
  constexpr int D = R == 1 ? 4 : 2;
  const int first_task = cta * kWarps + warp;
  const int my_tasks = first_task < a.tasks ? (a.tasks - 1 - first_task) / task_stride + 1 : 0;
  const int nsteps = my_tasks * iters;
  Rows ld_rows, cp_rows;
  Tile ring[D];
  int ld_step = 0, ld_task = first_task, ld_it = 0;
  auto issue = [&](Tile& d) {
    if (ld_step >= nsteps) return;
    if (ld_it == 0) open_task(ld_task, ld_rows);
    load_tile(ld_rows, ld_it, d);
    ++ld_step;
    if (++ld_it == iters) {
      ld_it = 0;
      ld_task += task_stride;
    }
  };
#pragma unroll
  for (int j = 0; j < D; ++j) issue(ring[j]);
  wait();
  if (M == 1 && a.pre_op != 0) {
    mlx_stage_x_pre<MODE>(a, xs, xc, cta);
  } else {
    mlx_stage_x<M, MODE>(a, xs, xc);
  }
  if (nsteps == 0) return;

  float acc[R][M];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

  int cp_task = first_task, cp_it = 0;
  open_task(cp_task, cp_rows);
  for (int s0 = 0; s0 < nsteps; s0 += D) {
#pragma unroll
    for (int j = 0; j < D; ++j) {
      if (s0 + j >= nsteps) break;
      const Tile cur = ring[j];
      issue(ring[j]);  // the slot's next occupant: step s0 + j + D
      const int it = cp_it;
      float2 F[R][M];
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) F[r][m] = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float4 xa[M], xb[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4* base = xs + ((size_t)(m * iters + it) * 8 + 2 * k) * 32 + lane;
          xa[m] = base[0];
          xb[m] = base[32];
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          uint32_t word = k == 0 ? cur.w[r].x : k == 1 ? cur.w[r].y : k == 2 ? cur.w[r].z : cur.w[r].w;
          float f[8];
          Unpack<MODE>::run(word, f);
#pragma unroll
          for (int m = 0; m < M; ++m) {
            fma2(F[r][m], make_float2(f[0], f[1]), make_float2(xa[m].x, xa[m].y));
            fma2(F[r][m], make_float2(f[2], f[3]), make_float2(xa[m].z, xa[m].w));
            fma2(F[r][m], make_float2(f[4], f[5]), make_float2(xb[m].x, xb[m].y));
            fma2(F[r][m], make_float2(f[6], f[7]), make_float2(xb[m].z, xb[m].w));
          }
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float2 c = xc[(m * iters + it) * 32 + lane];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float dot = (F[r][m].x + F[r][m].y) - c.x;
          acc[r][m] = fmaf(tile_scale(cur.sb[r]), dot, acc[r][m]);
          acc[r][m] = fmaf(tile_bias(cur.sb[r]), c.y, acc[r][m]);
        }
      }
      if (++cp_it == iters) {  // the task's rows are complete
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) {
            float v = warp_sum(acc[r][m]);
            acc[r][m] = 0.f;
            if (lane == 0 && cp_rows.row0 + r < cp_rows.rows && m < a.batch)
              cp_rows.out[(size_t)m * cp_rows.rows + cp_rows.row0 + r] = v;
          }
        cp_it = 0;
        cp_task += task_stride;
        if (s0 + j + 1 < nsteps) open_task(cp_task, cp_rows);
      }
    }
  }
}

// The product of a list entry (one row per warp task, batch 1), arranged so that as little as
// possible is left to do once x exists: the tiles of a warp's first four steps are loaded and the
// nibbles of its first two steps are already turned into floats while the producer of x is
// awaited; x is staged with one pass and one barrier, each lane forming its unit's two constants
// from the values it reads anyway.  Same arithmetic, in the same order, as mlx_gemv_body.
template <int MODE, bool SB_BF16, class Wait>
__device__ __forceinline__ void mlx_list_body(const MlxArgs& a, unsigned char* smem_raw, int cta, int nctas, Wait wait) {
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int task_stride = nctas * kWarps, iters = a.iters, units = a.units;
  typedef typename std::conditional<SB_BF16, uint32_t, float2>::type SbT;
  constexpr int D = 4, P = 2;
  struct Row {
    const uint4* w;
    const SbT* sb;
    float* out;  // where this task's result goes, or nullptr
  };
  struct Tile {
    uint4 w;
    SbT sb;
  };
  auto open_task = [&](int task, Row& t) {
    int seg = 0;
#pragma unroll
    for (int s = 1; s < kMaxSeg; ++s)
      if (s < a.nseg && task >= a.seg[s].task0) seg = s;
    const MlxSeg& sg = a.seg[seg];
    const int row = task - sg.task0;
    t.w = sg.w + (size_t)row * units;
    t.sb = reinterpret_cast<const SbT*>(sg.sb) + (size_t)row * a.groups;
    t.out = sg.out + row;
  };
  const int first_task = cta * kWarps + warp;
  const int my_tasks = first_task < a.tasks ? (a.tasks - 1 - first_task) / task_stride + 1 : 0;
  const int nsteps = my_tasks * iters;
  Row ld_row, cp_row;
  Tile ring[D];
  int ld_step = 0, ld_task = first_task, ld_it = 0;
  auto issue = [&](Tile& d) {
    if (ld_step >= nsteps) return;
    if (ld_it == 0) open_task(ld_task, ld_row);
    int unit = ld_it * 32 + lane;
    if (unit >= units) unit = units - 1;  // x is zero there; any finite weight will do
    d.w = ld_stream(ld_row.w + unit);
    d.sb = __ldg(ld_row.sb + (unit >> a.ug_shift));
    ++ld_step;
    if (++ld_it == iters) {
      ld_it = 0;
      ld_task += task_stride;
    }
  };
#pragma unroll
  for (int j = 0; j < D; ++j) issue(ring[j]);
  float pf[P][32];
#pragma unroll
  for (int p = 0; p < P; ++p)
    if (p < nsteps) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t word = k == 0 ? ring[p].w.x : k == 1 ? ring[p].w.y : k == 2 ? ring[p].w.z : ring[p].w.w;
        float f[8];
        Unpack<MODE>::run(word, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) pf[p][8 * k + e] = f[e];
      }
    }
  wait();
  if (a.pre_op != 0) {
    // residual add + RMSNorm, or SiLU(x) * b, applied while x is staged (as in goph_mlx_gemv_pre)
    mlx_stage_x_pre<MODE>(a, xs, reinterpret_cast<float2*>(smem_raw + (size_t)iters * 8 * 32 * 16), cta);
  } else {  // x -> shared memory, [iteration][slot][lane]; plain (coherent) loads
    const int slot = threadIdx.x & 7, u0 = threadIdx.x >> 3;  // consecutive threads, consecutive 16 bytes (see mlx_stage_x)
    for (int j0 = 0; j0 < iters; j0 += 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int unit = (j0 + u) * 32 + u0;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j0 + u < iters && unit < units) v[u] = *reinterpret_cast<const float4*>(a.x + (size_t)unit * 32 + slot * 4);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (j0 + u < iters) xs[((j0 + u) * 8 + slot) * 32 + u0] = v[u];
    }
    __syncthreads();
  }
  if (nsteps == 0) return;

  float acc = 0.f;
  int cp_task = first_task, cp_it = 0;
  open_task(cp_task, cp_row);
  // one step: F = sum (offset + nibble) * x over the lane's unit, then the scale and bias terms
  auto step = [&](auto&& nibbles, const SbT sb, int s) {
    float se = 0.f, so = 0.f;
    float2 F = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float4 xa = xs[(cp_it * 8 + 2 * k) * 32 + lane], xb = xs[(cp_it * 8 + 2 * k + 1) * 32 + lane];
      se += xa.x + xa.z;
      so += xa.y + xa.w;
      se += xb.x + xb.z;
      so += xb.y + xb.w;
      float f[8];
      nibbles(k, f);
      fma2(F, make_float2(f[0], f[1]), make_float2(xa.x, xa.y));
      fma2(F, make_float2(f[2], f[3]), make_float2(xa.z, xa.w));
      fma2(F, make_float2(f[4], f[5]), make_float2(xb.x, xb.y));
      fma2(F, make_float2(f[6], f[7]), make_float2(xb.z, xb.w));
    }
    const float2 c = mlx_unit_consts<MODE>(se, so);
    const float dot = (F.x + F.y) - c.x;
    float sc, bi;
    if constexpr (SB_BF16) {
      sc = __uint_as_float(sb << 16);
      bi = __uint_as_float(sb & 0xFFFF0000u);
    } else {
      sc = sb.x;
      bi = sb.y;
    }
    acc = fmaf(sc, dot, acc);
    acc = fmaf(bi, c.y, acc);
    if (++cp_it == iters) {  // the task's row is complete
      const float v = warp_sum(acc);
      acc = 0.f;
      if (lane == 0) *cp_row.out = v;
      cp_it = 0;
      cp_task += task_stride;
      if (s + 1 < nsteps) open_task(cp_task, cp_row);
    }
  };
#pragma unroll
  for (int p = 0; p < P; ++p)
    if (p < nsteps) {
      const SbT sb = ring[p].sb;
      issue(ring[p]);  // the slot's next occupant: step p + D
      step([&](int k, float (&f)[8]) {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = pf[p][8 * k + e];
      }, sb, p);
    }
  for (int s0 = P; s0 < nsteps; s0 += D) {
#pragma unroll
    for (int j = 0; j < D; ++j) {
      if (s0 + j >= nsteps) break;
      const Tile cur = ring[(P + j) % D];
      issue(ring[(P + j) % D]);
      step([&](int k, float (&f)[8]) {
        const uint32_t word = k == 0 ? cur.w.x : k == 1 ? cur.w.y : k == 2 ? cur.w.z : cur.w.w;
        Unpack<MODE>::run(word, f);
      }, cur.sb, s0 + j);
    }
  }
}

// One product per launch; x may come from the kernel in front (programmatic dependent launch).
template <int R, int M, int MODE, bool SB_BF16>
__global__ void __launch_bounds__(kThreads)
mlx_gemv_kernel(const __grid_constant__ MlxArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  mlx_gemv_body<R, M, MODE, SB_BF16>(a, smem_raw, blockIdx.x, gridDim.x,
                                     [] { asm volatile("griddepcontrol.wait;" ::: "memory"); });
}

// A list of products in one cooperative launch: every CTA works through the list, and a barrier
// over the whole grid stands between consecutive products (product k+1 may read what product k
// wrote).  Each CTA issues its first weight loads of product k+1 before it waits at the barrier,
// and fetches the next product's arguments while it computes.  The barrier is a counter in global
// memory that only grows: launch number L of a list of n products on G CTAs starts at L*(n-1)*G
// (L is read from launches[0] before a CTA's first arrival and advanced by CTA 0 after the last
// barrier, when every CTA has read it).  A wait gives up after about a second: the CTA records
// 200 + the product's index in *status and leaves the list, and so do the others.
constexpr long long kBarrierTimeoutCycles = 2000000000ll;

template <int R, int MODE, bool SB_BF16>
__global__ void __launch_bounds__(kThreads, 2)
mlx_program_kernel(const MlxArgs* __restrict__ ops, int nops, unsigned* counter, unsigned* launches, int* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(16) MlxArgs args[2];
  __shared__ unsigned s_base;
  __shared__ int s_abort;
  constexpr int kArgWords = sizeof(MlxArgs) / 4;
  static_assert(sizeof(MlxArgs) % 4 == 0, "MlxArgs is copied word by word");
  for (int i = threadIdx.x; i < kArgWords; i += kThreads)
    reinterpret_cast<uint32_t*>(&args[0])[i] = reinterpret_cast<const uint32_t*>(&ops[0])[i];
  if (threadIdx.x == 0) {
    s_base = *reinterpret_cast<volatile unsigned*>(launches) * (unsigned)(nops - 1) * gridDim.x;
    s_abort = 0;
  }
  __syncthreads();
  for (int op = 0; op < nops; ++op) {
    auto wait = [&] {
      // the next product's arguments, fetched by the upper half of the CTA while thread 0 polls;
      // they become visible to all with the barriers inside the staging of x
      if (op + 1 < nops && threadIdx.x >= 128) {
        for (int i = threadIdx.x - 128; i < kArgWords; i += kThreads - 128)
          reinterpret_cast<uint32_t*>(&args[(op + 1) & 1])[i] = reinterpret_cast<const uint32_t*>(&ops[op + 1])[i];
      }
      if (op == 0) return;
      if (threadIdx.x == 0) {
        const unsigned target = s_base + (unsigned)op * gridDim.x;
        const long long t0 = clock64();
        unsigned seen;
        while (true) {
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
          if ((int)(seen - target) >= 0) break;
          if (clock64() - t0 > kBarrierTimeoutCycles) {
            s_abort = 1;
            atomicExch(status, 200 + op);
            break;
          }
        }
      }
      __syncthreads();
    };
    // R rows per warp task: one row at a time with the nibbles unpacked ahead (R == 1), or R rows
    // sharing every load of x (the streaming kernel's loop)
    if constexpr (R == 1) mlx_list_body<MODE, SB_BF16>(args[op & 1], smem_raw, blockIdx.x, gridDim.x, wait);
    else mlx_gemv_body<R, 1, MODE, SB_BF16>(args[op & 1], smem_raw, blockIdx.x, gridDim.x, wait);
    __syncthreads();  // every warp is done with x in shared memory and has stored its rows
    if (s_abort) return;
    if (op + 1 < nops && threadIdx.x == 0)
      asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(counter), "r"(1u) : "memory");
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && nops > 1) atomicAdd(launches, 1u);
}

// Any group size / ragged in_dim: one warp per row, plain conversions, x from global.
template <bool SB_BF16>
__global__ void __launch_bounds__(kThreads)
mlx_gemv_generic_kernel(const uint32_t* __restrict__ w, const void* __restrict__ sb,
                        const float* __restrict__ x, float* __restrict__ out, int out_dim, int in_dim,
                        int gs, int groups, int batch) {
  int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= out_dim) return;
  int words = in_dim / 8;
  for (int m = 0; m < batch; ++m) {
    const float* xm = x + (size_t)m * in_dim;
    float acc = 0.f;
    for (int j = lane; j < words; j += 32) {
      uint32_t q = w[(size_t)row * words + j];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int col = j * 8 + e;
        int g = col / gs;
        float s, b;
        if (SB_BF16) {
          uint32_t v = reinterpret_cast<const uint32_t*>(sb)[(size_t)row * groups + g];
          s = __uint_as_float(v << 16);
          b = __uint_as_float(v & 0xFFFF0000u);
        } else {
          float2 v = reinterpret_cast<const float2*>(sb)[(size_t)row * groups + g];
          s = v.x;
          b = v.y;
        }
        float xv = xm[col];
        acc = fmaf(s * (float)((q >> (4 * e)) & 0xF) + b, xv, acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) out[(size_t)m * out_dim + row] = acc;
  }
}

// mlx.DequantTo: one thread per packed word, float32(nibble)*scale then +bias, both
// rounded (the intrinsics forbid contraction into an FMA).
template <bool SB_BF16>
__global__ void mlx_dequant_kernel(const uint32_t* __restrict__ w, const void* __restrict__ sb,
                                   float* __restrict__ out, size_t total_words, int words_per_row,
                                   int gs, int groups) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_words) return;
  size_t row = i / words_per_row;
  int j = (int)(i - row * words_per_row);
  uint32_t q = w[i];
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    int g = (j * 8 + e) / gs;
    float s, b;
    if (SB_BF16) {
      uint32_t t = reinterpret_cast<const uint32_t*>(sb)[row * groups + g];
      s = __uint_as_float(t << 16);
      b = __uint_as_float(t & 0xFFFF0000u);
    } else {
      float2 t = reinterpret_cast<const float2*>(sb)[row * groups + g];
      s = t.x;
      b = t.y;
    }
    v[e] = __fadd_rn(__fmul_rn((float)((q >> (4 * e)) & 0xF), s), b);
  }
  float4* o = reinterpret_cast<float4*>(out + i * 8);
  o[0] = make_float4(v[0], v[1], v[2], v[3]);
  o[1] = make_float4(v[4], v[5], v[6], v[7]);
}

// mlx.DequantTo from the tiled layout (bf16 table, group size 64).
__global__ void mlx_dequant_tiled_kernel(const unsigned char* __restrict__ tiled, float* __restrict__ out,
                                         size_t total_words, int words_per_row, int nchunks) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_words) return;
  int row = (int)(i / words_per_row), j = (int)(i - (size_t)row * words_per_row);
  uint32_t q = *reinterpret_cast<const uint32_t*>(tiled + mlx_tiled_word_offset(row, j * 8, nchunks));
  uint32_t t = *reinterpret_cast<const uint32_t*>(tiled + mlx_tiled_meta_offset(row, j * 8, nchunks));
  float s = __uint_as_float(t << 16), b = __uint_as_float(t & 0xFFFF0000u);
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = __fadd_rn(__fmul_rn((float)((q >> (4 * e)) & 0xF), s), b);
  float4* o = reinterpret_cast<float4*>(out + i * 8);
  o[0] = make_float4(v[0], v[1], v[2], v[3]);
  o[1] = make_float4(v[4], v[5], v[6], v[7]);
}

// Upload helpers: decide whether every scale/bias is a bf16 value, then interleave.
__global__ void mlx_sb_probe_kernel(const float* __restrict__ s, const float* __restrict__ b, size_t n,
                                    int* __restrict__ not_bf16) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if ((__float_as_uint(s[i]) & 0xFFFFu) | (__float_as_uint(b[i]) & 0xFFFFu)) *not_bf16 = 1;
}

__global__ void mlx_sb_pack_kernel(const float* __restrict__ s, const float* __restrict__ b, size_t n,
                                   void* __restrict__ dst, int as_bf16) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (as_bf16)
    reinterpret_cast<uint32_t*>(dst)[i] = (__float_as_uint(s[i]) >> 16) | (__float_as_uint(b[i]) & 0xFFFF0000u);
  else
    reinterpret_cast<float2*>(dst)[i] = make_float2(s[i], b[i]);
}

// ---- host side ------------------------------------------------------------------

typedef void (*MlxKernel)(const MlxArgs);

template <int R, int M, int MODE>
static MlxKernel pick_sb(bool bf16) {
  return bf16 ? (MlxKernel)mlx_gemv_kernel<R, M, MODE, true> : (MlxKernel)mlx_gemv_kernel<R, M, MODE, false>;
}

template <int R, int M>
static MlxKernel pick_mode(int mode, bool bf16) {
  if (M == 1) {
    if (mode == UNPACK_PAIR) return pick_sb<R, M, (M == 1 ? UNPACK_PAIR : UNPACK_EXACT)>(bf16);
    if (mode == UNPACK_CVT) return pick_sb<R, M, (M == 1 ? UNPACK_CVT : UNPACK_EXACT)>(bf16);
  }
  return pick_sb<R, M, UNPACK_EXACT>(bf16);
}

static MlxKernel pick_kernel(int R, int M, int mode, bool bf16) {
  switch (M) {
    case 1:
      return R == 4 ? pick_mode<4, 1>(mode, bf16) : R == 2 ? pick_mode<2, 1>(mode, bf16) : pick_mode<1, 1>(mode, bf16);
    case 2:
      return R == 4 ? pick_mode<4, 2>(mode, bf16) : R == 2 ? pick_mode<2, 2>(mode, bf16) : pick_mode<1, 2>(mode, bf16);
    case 4:
      return R == 4 ? pick_mode<4, 4>(mode, bf16) : R == 2 ? pick_mode<2, 4>(mode, bf16) : pick_mode<1, 4>(mode, bf16);
    default:
      return R >= 2 ? pick_mode<2, 8>(mode, bf16) : pick_mode<1, 8>(mode, bf16);
  }
}

static bool valid_handle(const goph_mlx_weight* w) {
  return w && w->magic == kMagicMLX && (w->tiled || (w->qweight && w->sb)) && w->in_dim > 0 && w->out_dim > 0 &&
         w->group_size > 0 && w->groups == w->in_dim / w->group_size;
}

static bool fast_path_ok(const goph_mlx_weight* w) {
  int gs = w->group_size;
  return w->in_dim % 32 == 0 && gs >= 32 && (gs & (gs - 1)) == 0;
}

// One launch of the streaming kernel for up to kMaxSeg weights sharing x, batch <= 8.
struct MlxPre {
  int op = 0;
  const float* b = nullptr;
  const float* w = nullptr;
  float* hidden = nullptr;
  float eps = 0.f;
};

static int launch_stream(const goph_mlx_weight* const* ws, float* const* outs, int n, const float* x,
                         int batch, cudaStream_t stream, const MlxPre* pre = nullptr) {
  const goph_mlx_weight* w0 = ws[0];
  DeviceState& st = device_state(w0->device);
  MlxArgs a;
  memset(&a, 0, sizeof a);
  a.nseg = n;
  a.x = x;
  a.batch = batch;
  a.in_dim = w0->in_dim;
  a.units = w0->in_dim / 32;
  a.iters = (a.units + 31) / 32;
  a.groups = w0->groups;
  int upg = w0->group_size / 32, sh = 0;
  while ((1 << sh) < upg) ++sh;
  a.ug_shift = sh;
  a.x_aligned = ((uintptr_t)x % 16) == 0;
  if (pre) {
    a.pre_op = pre->op;
    a.pre_b = pre->b;
    a.pre_w = pre->w;
    a.pre_hidden = pre->hidden;
    a.pre_eps = pre->eps;
  }

  int M = batch <= 1 ? 1 : batch <= 2 ? 2 : batch <= 4 ? 4 : 8;
  long total_rows = 0;
  for (int i = 0; i < n; ++i) total_rows += ws[i]->out_dim;
  // Rows per warp.  Batches: as many as keep every SM's 16 resident warps busy for two rounds.
  // Batch 1 is latency-bound (every CTA stages the whole x, and a launch costs by the CTA): two rows per
  // warp from 512 rows on.  Measured on the Qwen3-0.6B decode step (145 dependent launches per token,
  // prompt positions): 1250 tok/s with one row per warp, 1400-1440 with two, 1330 with four, 1190 with
  // four for the wide and two for the deep projections.
  int R = options().mlx_rows;
  if (R != 1 && R != 2 && R != 4) {
    if (M == 1) {
      R = total_rows >= 512 ? 2 : 1;
    } else {
      long want = (long)st.sm_count * 2 * kWarps * 2;
      R = total_rows / 4 >= want ? 4 : total_rows / 2 >= want ? 2 : 1;
    }
  }
  if (M == 8 && R == 4) R = 2;
  int tasks = 0;
  for (int i = 0; i < n; ++i) {
    a.seg[i].w = reinterpret_cast<const uint4*>(ws[i]->qweight);
    a.seg[i].sb = ws[i]->sb;
    a.seg[i].out = outs[i];
    a.seg[i].rows = ws[i]->out_dim;
    a.seg[i].task0 = tasks;
    tasks += (ws[i]->out_dim + R - 1) / R;
  }
  a.tasks = tasks;

  const int mode = options().mlx_unpack;
  MlxKernel k = pick_kernel(R, M, mode, w0->sb_bf16 != 0);
  size_t smem = mlx_smem_bytes(M, a.iters);
  GOPH_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int per_sm = 0;
  GOPH_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, kThreads, smem));
  if (per_sm < 1) return fail(GOPH_E_UNSUPPORTED, "MLX GEMV kernel does not fit (smem %zu)", smem);
  int grid = (tasks + kWarps - 1) / kWarps;
  if (options().mlx_ctas_per_sm > 0 && per_sm > options().mlx_ctas_per_sm) per_sm = options().mlx_ctas_per_sm;
  int cap = st.sm_count * per_sm;
  if (grid > cap) grid = cap;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, k, a));
  return GOPH_OK;
}

static int launch_generic(const goph_mlx_weight* w, float* out, const float* x, int batch, cudaStream_t stream) {
  int grid = (w->out_dim + kWarps - 1) / kWarps;
  note_launch();
  if (w->sb_bf16)
    mlx_gemv_generic_kernel<true><<<grid, kThreads, 0, stream>>>(w->qweight, w->sb, x, out, w->out_dim, w->in_dim,
                                                                 w->group_size, w->groups, batch);
  else
    mlx_gemv_generic_kernel<false><<<grid, kThreads, 0, stream>>>(w->qweight, w->sb, x, out, w->out_dim, w->in_dim,
                                                                  w->group_size, w->groups, batch);
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

// Products for n weights sharing x [batch,in]; outs[i] is [batch,out_i].
static int mlx_products(int n, float* const* outs, const goph_mlx_weight* const* ws, const float* x, int batch,
                        cudaStream_t stream) {
  const goph_mlx_weight* w0 = ws[0];
  bool any_tiled = false;
  for (int i = 0; i < n; ++i) any_tiled = any_tiled || ws[i]->tiled;
  if (any_tiled) {
    // tiled weights run on the tensor cores; row-major ones in the same call take their own path
    bool prepared = false;  // weights of one call share x: its digits are prepared once
    for (int i = 0; i < n; ++i) {
      const goph_mlx_weight* one = ws[i];
      float* o = outs[i];
      int rc;
      if (one->tiled && batch > 8) {
        // more rows than one pass of the integer kernel takes: bf16 operands, weights streamed once
        // per 16 rows (general f32 activations are split into three exact bf16 pieces)
        rc = tc_gemm_mlx(one, o, x, false, batch, stream);
      } else if (one->tiled) {
        rc = mlx_mma_launch(one, o, x, batch, options().mlx_digits, stream, prepared);
        prepared = true;
      } else {
        rc = mlx_products(1, &o, &one, x, batch, stream);
      }
      if (rc) return rc;
    }
    return GOPH_OK;
  }
  bool uniform = true;
  for (int i = 0; i < n; ++i)
    uniform = uniform && fast_path_ok(ws[i]) && ws[i]->sb_bf16 == w0->sb_bf16;
  if (!uniform || n > kMaxSeg) {
    for (int i = 0; i < n; ++i) {
      const goph_mlx_weight* one = ws[i];
      float* o = outs[i];
      int rc = fast_path_ok(one) ? mlx_products(1, &o, &one, x, batch, stream)
                                 : launch_generic(one, o, x, batch, stream);
      if (rc) return rc;
    }
    return GOPH_OK;
  }
  int units = w0->in_dim / 32, iters = (units + 31) / 32;
  if (mlx_smem_bytes(1, iters) > (size_t)kSmemBudget) {
    for (int i = 0; i < n; ++i)
      if (int rc = launch_generic(ws[i], outs[i], x, batch, stream)) return rc;
    return GOPH_OK;
  }
  // Batch tile: the largest of 8/4/2/1 whose x fits in shared memory.
  int tile = 8;
  while (tile > 1 && mlx_smem_bytes(tile, iters) > (size_t)kSmemBudget) tile >>= 1;
  for (int b0 = 0; b0 < batch; b0 += tile) {
    int nb = batch - b0 < tile ? batch - b0 : tile;
    float* sub[kMaxSeg];
    for (int i = 0; i < n; ++i) sub[i] = outs[i] + (size_t)b0 * ws[i]->out_dim;
    if (int rc = launch_stream(ws, sub, n, x + (size_t)b0 * w0->in_dim, nb, stream)) return rc;
  }
  return GOPH_OK;
}

typedef void (*MlxProgramKernel)(const MlxArgs*, int, unsigned*, unsigned*, int*);

template <int R>
static MlxProgramKernel pick_program_kernel_r(int mode, bool bf16) {
  if (mode == UNPACK_PAIR) return bf16 ? mlx_program_kernel<R, UNPACK_PAIR, true> : mlx_program_kernel<R, UNPACK_PAIR, false>;
  if (mode == UNPACK_CVT) return bf16 ? mlx_program_kernel<R, UNPACK_CVT, true> : mlx_program_kernel<R, UNPACK_CVT, false>;
  return bf16 ? mlx_program_kernel<R, UNPACK_EXACT, true> : mlx_program_kernel<R, UNPACK_EXACT, false>;
}

static MlxProgramKernel pick_program_kernel(int rows, int mode, bool bf16) {
  return rows == 1 ? pick_program_kernel_r<1>(mode, bf16) : rows == 2 ? pick_program_kernel_r<2>(mode, bf16)
                                                                      : pick_program_kernel_r<4>(mode, bf16);
}

}  // namespace goph

// A fixed list of batch-1 products launched as one cooperative kernel (see mlx_program_kernel).
struct goph_mlx_program {
  uint32_t magic;
  int device;
  int nops;
  int grid;
  size_t smem;
  goph::MlxProgramKernel kernel;
  goph::MlxArgs* ops;   // device
  unsigned* words;      // device: [0] barrier counter, [1] launches so far, [2] status
};

using namespace goph;

constexpr uint32_t kMagicProgram = 0x4d50524f;  // "MPRO"

GOPH_API int goph_mlx_program_create_pre(int device, int n_ops, const int* weights_per_op,
                                         const goph_mlx_weight* const* ws, float* const* outs_dev,
                                         const float* const* xs_dev, const int* pre_ops, const float* const* pre_b,
                                         const float* const* pre_w, float* const* pre_hidden, const float* pre_eps,
                                         goph_mlx_program** out);

GOPH_API int goph_mlx_program_create(int device, int n_ops, const int* weights_per_op,
                                     const goph_mlx_weight* const* ws, float* const* outs_dev,
                                     const float* const* xs_dev, goph_mlx_program** out) {
  return goph_mlx_program_create_pre(device, n_ops, weights_per_op, ws, outs_dev, xs_dev, nullptr, nullptr, nullptr, nullptr,
                                     nullptr, out);
}

GOPH_API int goph_mlx_program_create_pre(int device, int n_ops, const int* weights_per_op,
                                         const goph_mlx_weight* const* ws, float* const* outs_dev,
                                         const float* const* xs_dev, const int* pre_ops, const float* const* pre_b,
                                         const float* const* pre_w, float* const* pre_hidden, const float* pre_eps,
                                         goph_mlx_program** out) {
  clear_error();
  if (!out) return fail(GOPH_E_INVALID, "goph_mlx_program_create: nil result pointer");
  *out = nullptr;
  if (n_ops <= 0 || !weights_per_op || !ws || !outs_dev || !xs_dev)
    return fail(GOPH_E_INVALID, "goph_mlx_program_create: empty list or nil array");
  std::vector<MlxArgs> ops((size_t)n_ops);
  int k = 0, max_iters = 1;
  // rows per warp task: one (the list's own loop with the nibbles unpacked ahead; measured best), or two
  // or four through option "mlx_rows" (the streaming kernel's loop: rows share every load of x)
  const int R = options().mlx_rows == 2 || options().mlx_rows == 4 ? options().mlx_rows : 1;
  const goph_mlx_weight* first = ws[0];
  for (int o = 0; o < n_ops; ++o) {
    const int n = weights_per_op[o];
    if (n <= 0 || n > kMaxSeg) return fail(GOPH_E_INVALID, "product %d: %d weights (1..%d allowed)", o, n, kMaxSeg);
    MlxArgs& a = ops[o];
    memset(&a, 0, sizeof a);
    const goph_mlx_weight* w0 = ws[k];
    for (int i = 0; i < n; ++i) {
      const goph_mlx_weight* w = ws[k + i];
      if (!valid_handle(w)) return fail(GOPH_E_INVALID, "product %d: invalid weight handle", o);
      if (w->device != device) return fail(GOPH_E_INVALID, "product %d: weight lives on device %d", o, w->device);
      if (w->tiled || !fast_path_ok(w))
        return fail(GOPH_E_UNSUPPORTED, "product %d: only row-major weights with a power-of-two group size >= 32 "
                                        "and in_dim %% 32 == 0 can join a product list", o);
      if (w->in_dim != w0->in_dim || w->group_size != w0->group_size)
        return fail(GOPH_E_INVALID, "product %d: its weights do not share x (in_dim/group size differ)", o);
      if (!first || w->sb_bf16 != first->sb_bf16)
        return fail(GOPH_E_UNSUPPORTED, "product %d: scale tables of one list must share a format", o);
      if (!outs_dev[k + i]) return fail(GOPH_E_INVALID, "product %d: nil output", o);
      a.seg[i].w = reinterpret_cast<const uint4*>(w->qweight);
      a.seg[i].sb = w->sb;
      a.seg[i].out = outs_dev[k + i];
      a.seg[i].rows = w->out_dim;
      a.seg[i].task0 = a.tasks;
      a.tasks += (w->out_dim + R - 1) / R;
    }
    if (!xs_dev[o] || (uintptr_t)xs_dev[o] % 16) return fail(GOPH_E_INVALID, "product %d: x is nil or not 16-byte aligned", o);
    // the barrier orders products against each other, not a product against itself: what a product
    // writes (outputs, the hidden vector of operation 1) must not meet what it reads
    const int pre_op = pre_ops ? pre_ops[o] : 0;
    const float* pb = pre_op && pre_b ? pre_b[o] : nullptr;
    const float* pw = pre_op && pre_w ? pre_w[o] : nullptr;
    float* ph = pre_op == 1 && pre_hidden ? pre_hidden[o] : nullptr;
    if (pre_op < 0 || pre_op > 2) return fail(GOPH_E_INVALID, "product %d: pre_op=%d", o, pre_op);
    if ((pre_op == 1 && !pw) || (pre_op == 2 && !pb)) return fail(GOPH_E_INVALID, "product %d: missing operand of its operation", o);
    if (((uintptr_t)pb | (uintptr_t)pw | (uintptr_t)ph) % 16) return fail(GOPH_E_INVALID, "product %d: vectors must be 16-byte aligned", o);
    {
      typedef std::pair<uintptr_t, uintptr_t> Range;
      auto range = [](const float* p, int n) { return Range((uintptr_t)p, (uintptr_t)(p + n)); };
      auto meet = [](Range p, Range q) { return p.first && q.first && p.first < q.second && q.first < p.second; };
      std::vector<Range> reads = {range(xs_dev[o], w0->in_dim), range(pb, w0->in_dim)}, writes = {range(ph, w0->in_dim)};
      for (int i = 0; i < n; ++i) writes.push_back(range(outs_dev[k + i], ws[k + i]->out_dim));
      for (const Range& wr : writes)
        for (const Range& rd : reads)
          if (meet(wr, rd)) return fail(GOPH_E_INVALID, "product %d: an output overlaps its x", o);
      for (size_t i = 0; i < writes.size(); ++i)
        for (size_t j = i + 1; j < writes.size(); ++j)
          if (meet(writes[i], writes[j])) return fail(GOPH_E_INVALID, "product %d: two of its outputs overlap", o);
    }
    a.pre_op = pre_op;
    a.pre_b = pb;
    a.pre_w = pw;
    a.pre_hidden = ph;
    a.pre_eps = pre_eps ? pre_eps[o] : 0.f;
    a.nseg = n;
    a.x = xs_dev[o];
    a.batch = 1;
    a.in_dim = w0->in_dim;
    a.units = w0->in_dim / 32;
    a.iters = (a.units + 31) / 32;
    a.groups = w0->groups;
    int upg = w0->group_size / 32, sh = 0;
    while ((1 << sh) < upg) ++sh;
    a.ug_shift = sh;
    a.x_aligned = 1;
    if (a.iters > max_iters) max_iters = a.iters;
    k += n;
  }
  const size_t smem = mlx_smem_bytes(1, max_iters);
  if (smem > (size_t)kSmemBudget) return fail(GOPH_E_UNSUPPORTED, "product list: in_dim too large for shared memory");
  if (int rc = use_device(device)) return rc;
  DeviceState& st = device_state(device);
  MlxProgramKernel kern = pick_program_kernel(R, options().mlx_unpack, first->sb_bf16 != 0);
  GOPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int per_sm = 0;
  GOPH_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem));
  if (per_sm < 1) return fail(GOPH_E_UNSUPPORTED, "product list kernel does not fit (smem %zu)", smem);
  if (per_sm > 2) per_sm = 2;  // 16 warps per SM keep the loads in flight; more CTAs only lengthen the barrier
  if (options().mlx_ctas_per_sm > 0 && per_sm > options().mlx_ctas_per_sm) per_sm = options().mlx_ctas_per_sm;
  auto* p = new goph_mlx_program();
  p->magic = kMagicProgram;
  p->device = device;
  p->nops = n_ops;
  p->grid = st.sm_count * per_sm;
  p->smem = smem;
  p->kernel = kern;
  cudaError_t e = cudaMalloc(&p->ops, ops.size() * sizeof(MlxArgs));
  if (e == cudaSuccess) e = cudaMalloc(&p->words, 64 + 48 * 8);
  if (e == cudaSuccess) e = cudaMemcpy(p->ops, ops.data(), ops.size() * sizeof(MlxArgs), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(p->words, 0, 64 + 48 * 8);
  if (e != cudaSuccess) {
    cudaFree(p->ops);
    cudaFree(p->words);
    delete p;
    return fail_cuda(e, "goph_mlx_program_create");
  }
  *out = p;
  return GOPH_OK;
}

GOPH_API int goph_mlx_program_run(goph_mlx_program* p, void* stream) {
  clear_error();
  if (!p || p->magic != kMagicProgram) return fail(GOPH_E_INVALID, "invalid product list handle");
  if (int rc = use_device(p->device)) return rc;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeCooperative;
  attr.val.cooperative = 1;  // every CTA resident at once: the barrier between products needs it
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(p->grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = p->smem;
  cfg.stream = (cudaStream_t)stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  // the attribute belongs to the kernel, not to the list: a list created later on the same
  // instantiation with a smaller request would otherwise leave this one without its shared memory
  GOPH_CUDA(cudaFuncSetAttribute(p->kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p->smem));
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, p->kernel, (const MlxArgs*)p->ops, p->nops, p->words, p->words + 1,
                               reinterpret_cast<int*>(p->words + 2)));
  return GOPH_OK;
}

GOPH_API int goph_mlx_program_status(goph_mlx_program* p, int* out_status) {
  clear_error();
  if (!p || p->magic != kMagicProgram) return fail(GOPH_E_INVALID, "invalid product list handle");
  if (!out_status) return fail(GOPH_E_INVALID, "goph_mlx_program_status: nil result pointer");
  if (int rc = use_device(p->device)) return rc;
  GOPH_CUDA(cudaMemcpy(out_status, p->words + 2, 4, cudaMemcpyDeviceToHost));
  return GOPH_OK;
}

GOPH_API int goph_mlx_program_free(goph_mlx_program* p) {
  clear_error();
  if (!p) return GOPH_OK;
  if (p->magic != kMagicProgram) return fail(GOPH_E_INVALID, "goph_mlx_program_free: not a product list handle");
  if (int rc = use_device(p->device)) return rc;
  cudaFree(p->ops);
  cudaFree(p->words);
  p->magic = 0;
  delete p;
  return GOPH_OK;
}

static int mlx_upload_common(int device, const uint32_t* weight, const float* scales, const float* biases,
                             bool on_device, int in_dim, int out_dim, int gs, goph_mlx_weight** out) {
  uint64_t groups = (uint64_t)in_dim / gs, want_w, want_s;
  mul_ok((uint64_t)out_dim, (uint64_t)in_dim / 8, &want_w);
  mul_ok((uint64_t)out_dim, groups, &want_s);
  goph_mlx_weight* h = new goph_mlx_weight();
  h->magic = kMagicMLX;
  h->device = device;
  h->in_dim = in_dim;
  h->out_dim = out_dim;
  h->group_size = gs;
  h->groups = (int)groups;
  h->tiled = nullptr;
  float *ds = nullptr, *db = nullptr;
  int* flag = nullptr;
  auto cleanup = [&](int rc) {
    if (!on_device) {
      cudaFree(ds);
      cudaFree(db);
    }
    cudaFree(flag);
    if (rc) {
      cudaFree(h->qweight);
      cudaFree(h->sb);
      cudaFree(h->tiled);
      delete h;
    }
    return rc;
  };
#define UP(call)                                            \
  do {                                                      \
    cudaError_t _e = (call);                                \
    if (_e != cudaSuccess) return cleanup(fail_cuda(_e, #call)); \
  } while (0)
  UP(cudaMalloc(&h->qweight, want_w * 4));
  UP(cudaMemcpy(h->qweight, weight, want_w * 4, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
  if (on_device) {
    ds = const_cast<float*>(scales);
    db = const_cast<float*>(biases);
  } else {
    UP(cudaMalloc(&ds, want_s * 4));
    UP(cudaMalloc(&db, want_s * 4));
    UP(cudaMemcpy(ds, scales, want_s * 4, cudaMemcpyHostToDevice));
    UP(cudaMemcpy(db, biases, want_s * 4, cudaMemcpyHostToDevice));
  }
  UP(cudaMalloc(&flag, sizeof(int)));
  UP(cudaMemset(flag, 0, sizeof(int)));
  unsigned blocks = (unsigned)((want_s + 255) / 256);
  mlx_sb_probe_kernel<<<blocks, 256>>>(ds, db, want_s, flag);
  int not_bf16 = 0;
  UP(cudaMemcpy(&not_bf16, flag, sizeof(int), cudaMemcpyDeviceToHost));
  h->sb_bf16 = not_bf16 ? 0 : 1;
  UP(cudaMalloc(&h->sb, want_s * (h->sb_bf16 ? 4 : 8)));
  mlx_sb_pack_kernel<<<blocks, 256>>>(ds, db, want_s, h->sb, h->sb_bf16);
  UP(cudaGetLastError());
  UP(cudaDeviceSynchronize());
#undef UP
  h->bytes = want_w * 4 + want_s * (h->sb_bf16 ? 4 : 8);
  // Tiled layout + tensor-core kernel for matrices large enough to amortise that kernel's fixed
  // cost (TMEM set-up, activation preparation, pipeline fill); small ones stay row-major.
  const bool big = (uint64_t)out_dim * (uint64_t)in_dim >= (8u << 20);
  if (mlx_mma_supported(h) && (options().mlx_layout == 2 || (options().mlx_layout == 0 && big))) {
    if (int rc = mlx_mma_make_tiled(h)) return cleanup(rc);
    cudaFree(h->qweight);
    cudaFree(h->sb);
    h->qweight = nullptr;
    h->sb = nullptr;
  }
  *out = h;
  return cleanup(GOPH_OK);
}

// validateMLXUploadInputs (backends/nvidia/runtime/mlx.go:34-55).
static int mlx_validate_dims(int in_dim, int out_dim, int gs) {
  if (in_dim <= 0 || out_dim <= 0 || gs <= 0 || in_dim % gs != 0 || in_dim % 8 != 0)
    return fail(GOPH_E_INVALID, "invalid MLX dims inDim=%d outDim=%d groupSize=%d", in_dim, out_dim, gs);
  return GOPH_OK;
}

GOPH_API int goph_mlx_upload(int device, const uint32_t* weight, uint64_t weight_len, const float* scales,
                             const float* biases, uint64_t scale_len, int in_dim, int out_dim, int group_size,
                             goph_mlx_weight** out) {
  clear_error();
  if (!out) return fail(GOPH_E_INVALID, "goph_mlx_upload: nil result pointer");
  *out = nullptr;
  if (int rc = mlx_validate_dims(in_dim, out_dim, group_size)) return rc;
  uint64_t want_w, want_s;
  if (!mul_ok((uint64_t)out_dim, (uint64_t)in_dim / 8, &want_w) ||
      !mul_ok((uint64_t)out_dim, (uint64_t)(in_dim / group_size), &want_s) || want_w > (UINT64_MAX >> 3))
    return fail(GOPH_E_INVALID, "MLX weight size overflow outDim=%d inDim=%d", out_dim, in_dim);
  if (!weight || weight_len < want_w)
    return fail(GOPH_E_INVALID, "weight length=%llu, want at least %llu", (unsigned long long)weight_len,
                (unsigned long long)want_w);
  if (!scales || !biases || scale_len < want_s)
    return fail(GOPH_E_INVALID, "scale/bias length=%llu, want at least %llu", (unsigned long long)scale_len,
                (unsigned long long)want_s);
  if (int rc = use_device(device)) return rc;
  return mlx_upload_common(device, weight, scales, biases, false, in_dim, out_dim, group_size, out);
}

GOPH_API int goph_mlx_upload_dev(int device, const uint32_t* weight_dev, const float* scales_dev,
                                 const float* biases_dev, int in_dim, int out_dim, int group_size,
                                 goph_mlx_weight** out) {
  clear_error();
  if (!out) return fail(GOPH_E_INVALID, "goph_mlx_upload_dev: nil result pointer");
  *out = nullptr;
  if (int rc = mlx_validate_dims(in_dim, out_dim, group_size)) return rc;
  uint64_t want_w;
  if (!mul_ok((uint64_t)out_dim, (uint64_t)in_dim / 8, &want_w) || want_w > (UINT64_MAX >> 3))
    return fail(GOPH_E_INVALID, "MLX weight size overflow outDim=%d inDim=%d", out_dim, in_dim);
  if (!weight_dev || !scales_dev || !biases_dev) return fail(GOPH_E_INVALID, "goph_mlx_upload_dev: nil buffer");
  if (int rc = use_device(device)) return rc;
  return mlx_upload_common(device, weight_dev, scales_dev, biases_dev, true, in_dim, out_dim, group_size, out);
}

GOPH_API int goph_mlx_free(goph_mlx_weight* w) {
  clear_error();
  if (!w) return GOPH_OK;
  if (w->magic != kMagicMLX) return fail(GOPH_E_INVALID, "goph_mlx_free: not an MLX weight handle");
  if (int rc = use_device(w->device)) return rc;
  cudaFree(w->qweight);
  cudaFree(w->sb);
  cudaFree(w->tiled);
  w->magic = 0;
  delete w;
  return GOPH_OK;
}

GOPH_API int goph_kernel_status(int device, int* out_status) {
  clear_error();
  if (!out_status) return fail(GOPH_E_INVALID, "goph_kernel_status: nil result pointer");
  if (int rc = use_device(device)) return rc;
  *out_status = mlx_mma_status(device);
  if (*out_status == 0) *out_status = tc_gemm_status(device);
  if (*out_status == 0) *out_status = fp8_mma_status(device);
  if (*out_status == 0) *out_status = gguf_work_status(device);
  if (*out_status == 0) *out_status = moe_status(device);
  if (*out_status == 0) *out_status = decode_ops_status();
  return GOPH_OK;
}

GOPH_API int goph_kernel_status_clear(int device) {
  clear_error();
  if (int rc = use_device(device)) return rc;
  GOPH_CUDA(cudaDeviceSynchronize());
  mlx_mma_status_clear(device);
  tc_gemm_status_clear(device);
  fp8_mma_status_clear(device);
  gguf_work_status_clear(device);
  moe_status_clear(device);
  decode_ops_status_clear();
  return GOPH_OK;
}

GOPH_API uint64_t goph_mlx_resident_bytes(const goph_mlx_weight* w) {
  return (w && w->magic == kMagicMLX) ? w->bytes : 0;
}

GOPH_API int goph_mlx_dequant(const goph_mlx_weight* w, float* out_dev, uint64_t out_len, void* stream) {
  clear_error();
  if (!valid_handle(w)) return fail(GOPH_E_INVALID, "goph_mlx_dequant: invalid weight handle");
  uint64_t need = (uint64_t)w->out_dim * w->in_dim;
  if (!out_dev || out_len < need)
    return fail(GOPH_E_INVALID, "dequant out length=%llu, want at least %llu", (unsigned long long)out_len,
                (unsigned long long)need);
  if ((uintptr_t)out_dev % 16) return fail(GOPH_E_INVALID, "dequant out must be 16-byte aligned");
  if (int rc = use_device(w->device)) return rc;
  size_t words = (size_t)w->out_dim * (w->in_dim / 8);
  unsigned blocks = (unsigned)((words + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (w->tiled)
    mlx_dequant_tiled_kernel<<<blocks, 256, 0, s>>>(w->tiled, out_dev, words, w->in_dim / 8, w->in_dim / 256);
  else if (w->sb_bf16)
    mlx_dequant_kernel<true><<<blocks, 256, 0, s>>>(w->qweight, w->sb, out_dev, words, w->in_dim / 8,
                                                    w->group_size, w->groups);
  else
    mlx_dequant_kernel<false><<<blocks, 256, 0, s>>>(w->qweight, w->sb, out_dev, words, w->in_dim / 8,
                                                     w->group_size, w->groups);
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

GOPH_API int goph_mlx_gemm_multi(int n, float* const* outs_dev, const goph_mlx_weight* const* ws,
                                 const float* x_dev, uint64_t x_len, int batch, void* stream) {
  clear_error();
  if (n <= 0 || n > kMaxSeg || !outs_dev || !ws) return fail(GOPH_E_INVALID, "goph_mlx_gemm_multi: n=%d out of 1..%d", n, kMaxSeg);
  if (batch <= 0) return fail(GOPH_E_INVALID, "goph_mlx_gemm_multi: batch=%d", batch);
  for (int i = 0; i < n; ++i) {
    if (!valid_handle(ws[i]) || !outs_dev[i]) return fail(GOPH_E_INVALID, "goph_mlx_gemm_multi: invalid weight or out %d", i);
    if (ws[i]->device != ws[0]->device || ws[i]->in_dim != ws[0]->in_dim || ws[i]->group_size != ws[0]->group_size)
      return fail(GOPH_E_INVALID, "goph_mlx_gemm_multi: weights %d and 0 differ in device/inDim/groupSize", i);
  }
  uint64_t need_x;
  if (!mul_ok((uint64_t)batch, (uint64_t)ws[0]->in_dim, &need_x) || !x_dev || x_len < need_x)
    return fail(GOPH_E_INVALID, "x length=%llu, want at least %llu", (unsigned long long)x_len,
                (unsigned long long)((uint64_t)batch * ws[0]->in_dim));
  if (int rc = use_device(ws[0]->device)) return rc;
  return mlx_products(n, outs_dev, ws, x_dev, batch, (cudaStream_t)stream);
}

GOPH_API int goph_mlx_gemm(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                           const goph_mlx_weight* w, int batch, void* stream) {
  clear_error();
  if (!valid_handle(w)) return fail(GOPH_E_INVALID, "invalid MLX weight handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)w->out_dim, &need_o) || !out_dev || out_len < need_o)
    return fail(GOPH_E_INVALID, "out length=%llu, want at least %llu", (unsigned long long)out_len,
                (unsigned long long)((uint64_t)batch * w->out_dim));
  return goph_mlx_gemm_multi(1, &out_dev, &w, x_dev, x_len, batch, stream);
}

GOPH_API int goph_mlx_gemm_bf16(float* out_dev, uint64_t out_len, const uint16_t* x_bf16_dev, uint64_t x_len,
                                const goph_mlx_weight* w, int batch, void* stream) {
  clear_error();
  if (!valid_handle(w)) return fail(GOPH_E_INVALID, "invalid MLX weight handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_x, need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)w->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)w->out_dim, &need_o))
    return fail(GOPH_E_INVALID, "batch size overflow");
  if (!x_bf16_dev || x_len < need_x || !out_dev || out_len < need_o)
    return fail(GOPH_E_INVALID, "buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len, (unsigned long long)need_x,
                (unsigned long long)out_len, (unsigned long long)need_o);
  if (!w->tiled)
    return fail(GOPH_E_UNSUPPORTED,
                "goph_mlx_gemm_bf16 needs a weight in the tiled layout (group size 64, in_dim a multiple of 256, "
                "uploaded with mlx_layout 0 or 2); this one is row-major");
  if (int rc = use_device(w->device)) return rc;
  return tc_gemm_mlx(w, out_dev, x_bf16_dev, true, batch, (cudaStream_t)stream);
}

GOPH_API int goph_mlx_gemv(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                           const goph_mlx_weight* w, void* stream) {
  return goph_mlx_gemm(out_dev, out_len, x_dev, x_len, w, 1, stream);
}

GOPH_API int goph_mlx_gemm_host(float* out_host, uint64_t out_len, const float* x_host, uint64_t x_len,
                                const goph_mlx_weight* w, int batch) {
  clear_error();
  if (!valid_handle(w)) return fail(GOPH_E_INVALID, "invalid MLX weight handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_x, need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)w->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)w->out_dim, &need_o))
    return fail(GOPH_E_INVALID, "batch size overflow");
  if (!x_host || x_len < need_x || !out_host || out_len < need_o)
    return fail(GOPH_E_INVALID, "host buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len,
                (unsigned long long)need_x, (unsigned long long)out_len, (unsigned long long)need_o);
  if (int rc = use_device(w->device)) return rc;
  float *dx = nullptr, *dout = nullptr;
  GOPH_CUDA(cudaMalloc(&dx, need_x * 4));
  cudaError_t e = cudaMalloc(&dout, need_o * 4);
  if (e != cudaSuccess) {
    cudaFree(dx);
    return fail_cuda(e, "cudaMalloc(out)");
  }
  int rc = GOPH_OK;
  e = cudaMemcpy(dx, x_host, need_x * 4, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) rc = fail_cuda(e, "cudaMemcpy(x)");
  if (!rc) rc = goph_mlx_gemm(dout, need_o, dx, need_x, w, batch, nullptr);
  if (!rc) {
    e = cudaMemcpy(out_host, dout, need_o * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) rc = fail_cuda(e, "cudaMemcpy(out)");
  }
  cudaFree(dx);
  cudaFree(dout);
  return rc;
}


// out = W . f(x): the operation in front of a projection folded into the kernel that stages x
// (one launch instead of two in the decode step).  pre_op 1: v = x (+ b); hidden_out = v;
// f = RMSNorm(v) * norm_w.  pre_op 2: f = silu(x) * b.  Row-major weights of the CUDA-core kernel,
// batch 1; anything else is GOPH_E_UNSUPPORTED and the caller runs the two operations separately.
GOPH_API int goph_mlx_gemv_pre(float* out_dev, uint64_t out_len, const goph_mlx_weight* w, int pre_op, const float* x_dev,
                               const float* b_dev, const float* norm_w_dev, float* hidden_out_dev, float eps, void* stream) {
  clear_error();
  if (!valid_handle(w)) return fail(GOPH_E_INVALID, "goph_mlx_gemv_pre: invalid weight handle");
  if (pre_op != 1 && pre_op != 2) return fail(GOPH_E_INVALID, "goph_mlx_gemv_pre: pre_op=%d", pre_op);
  if (!out_dev || out_len < (uint64_t)w->out_dim || !x_dev) return fail(GOPH_E_INVALID, "goph_mlx_gemv_pre: buffers");
  if ((pre_op == 1 && !norm_w_dev) || (pre_op == 2 && !b_dev)) return fail(GOPH_E_INVALID, "goph_mlx_gemv_pre: missing operand");
  if (pre_op == 1 && hidden_out_dev && (hidden_out_dev == x_dev || hidden_out_dev == b_dev))
    return fail(GOPH_E_INVALID, "goph_mlx_gemv_pre: hidden_out must not alias an input (every CTA reads the inputs)");
  if (w->tiled || !fast_path_ok(w)) return fail(GOPH_E_UNSUPPORTED, "goph_mlx_gemv_pre: row-major weights with group size >= 32 only");
  const uintptr_t al = (uintptr_t)x_dev | (uintptr_t)b_dev | (uintptr_t)norm_w_dev | (uintptr_t)hidden_out_dev;
  if (al % 16) return fail(GOPH_E_INVALID, "goph_mlx_gemv_pre: vectors must be 16-byte aligned");
  if (int rc = use_device(w->device)) return rc;
  MlxPre pre;
  pre.op = pre_op;
  pre.b = b_dev;
  pre.w = norm_w_dev;
  pre.hidden = hidden_out_dev;
  pre.eps = eps;
  return launch_stream(&w, &out_dev, 1, x_dev, 1, (cudaStream_t)stream, &pre);
}
