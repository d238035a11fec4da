// Streaming GEMV / small-batch skeleton shared by the GGUF and FP8 formats.
//
// Same shape as the MLX kernel: a warp owns R rows at a time; lane l of iteration `it`
// owns one 16-byte unit (unit = 32*it + l) of each of those rows, so a warp instruction is
// a 512-byte coalesced, L1-bypassing load per row.  x is staged once per CTA in shared
// memory as f32 in the order [batch][it][slot][lane] (conflict-free LDS.128), with one
// float2 of per-unit constants beside it when the format needs them (offset removal and
// the affine term).  The next step's weights are in flight while the current step computes.
//
// A format policy F provides:
//   kSlots                 float4 of x per unit (unit elements / 4)
//   kHasConsts             whether per-unit constants are needed
//   struct Row             per-row data of one unit (the 16 weight bytes + metadata)
//   load(a,row,unit,Row&)  issue the loads of one unit of one row
//   consts(se,so)          float2 from the even/odd-position sums of the unit's x
//   dot(Row, xs, c, acc)   acc[m] += contribution of this unit, for m < M
//   finish(a,row,v)        per-row epilogue (row scale, bias)
#pragma once

#include "goph_internal.cuh"

namespace goph {

constexpr int kGWarps = 8;
constexpr int kGThreads = kGWarps * 32;

struct StreamArgs {
  const uint8_t* w;     // weight bytes
  const void* aux;      // format metadata (Q8_0: f16 scales; FP8: f32 row scales)
  const float* bias;    // FP8 bias or nullptr
  float* out;           // [batch][rows]
  const float* x;       // [batch][in_dim]
  int rows, in_dim, batch;
  int units;            // 16-byte units per row
  int iters;            // ceil(units / 32)
  int x_aligned;
  int row_bytes;

};

template <class F>
__host__ __device__ inline size_t stream_smem_bytes(int M, int iters) {
  return (size_t)M * iters * (F::kSlots * 32 * 16 + (F::kHasConsts ? 32 * 8 : 0));
}

template <class F, int R, int M>
__global__ void __launch_bounds__(kGThreads)
stream_gemv_kernel(const __grid_constant__ StreamArgs a) {
  constexpr int S = F::kSlots;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)M * a.iters * S * 32 * 16);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int iters = a.iters;
  const int tasks = (a.rows + R - 1) / R;
  const int task_stride = gridDim.x * kGWarps;
  int task = blockIdx.x * kGWarps + warp, it = 0;

  typename F::Row cur[R], nxt[R];
  auto load_tile = [&](int t, int i, typename F::Row (&dst)[R]) {
    int unit = i * 32 + lane;
    if (unit >= a.units) unit = a.units - 1;  // x is zero there
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int row = t * R + r;
      if (row >= a.rows) row = a.rows - 1;
      F::load(a, row, unit, dst[r]);
    }
  };
  const bool has_work = task < tasks;
  if (has_work) load_tile(task, 0, cur);

  // ---- stage x ----
  {
    const int per_m = iters * S * 32, total = M * per_m;
    for (int idx = threadIdx.x; idx < total; idx += kGThreads) {
      int m = idx / per_m, rem = idx - m * per_m;
      int i = rem / (S * 32), slot = (rem >> 5) % S, l = rem & 31;
      int unit = i * 32 + l;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < a.batch && unit < a.units) {
        const float* p = a.x + (size_t)m * a.in_dim + (size_t)unit * (S * 4) + slot * 4;
        if (a.x_aligned)
          v = __ldg(reinterpret_cast<const float4*>(p));
        else
          v = make_float4(__ldg(p), __ldg(p + 1), __ldg(p + 2), __ldg(p + 3));
      }
      xs[idx] = v;
    }
    __syncthreads();
    if (F::kHasConsts) {
      const int nsum = M * iters * 32;
      for (int idx = threadIdx.x; idx < nsum; idx += kGThreads) {
        int mi = idx >> 5, l = idx & 31;
        float se = 0.f, so = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) {
          float4 v = xs[(mi * S + s) * 32 + l];
          se += v.x + v.z;
          so += v.y + v.w;
        }
        xc[idx] = F::consts(se, so);
      }
      __syncthreads();
    }
  }
  if (!has_work) return;

  float acc[R][M];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

  while (true) {
    int ntask = task, nit = it + 1;
    if (nit == iters) {
      nit = 0;
      ntask = task + task_stride;
    }
    const bool more = ntask < tasks;
    if (more) load_tile(ntask, nit, nxt);

    float4 xv[M][S];
    float2 c[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
      for (int s = 0; s < S; ++s) xv[m][s] = xs[((size_t)(m * iters + it) * S + s) * 32 + lane];
      c[m] = F::kHasConsts ? xc[(m * iters + it) * 32 + lane] : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) F::template dot<M>(cur[r], xv, c, acc[r]);

    if (it == iters - 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        int row = task * R + r;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float v = warp_sum(acc[r][m]);
          acc[r][m] = 0.f;
          if (lane == 0 && row < a.rows && m < a.batch) a.out[(size_t)m * a.rows + row] = F::finish(a, row, v);
        }
      }
    }
    if (!more) break;
#pragma unroll
    for (int r = 0; r < R; ++r) cur[r] = nxt[r];
    task = ntask;
    it = nit;
  }
}

typedef void (*StreamKernel)(const StreamArgs);

template <class F>
static StreamKernel stream_pick(int R, int M) {
  switch (M) {
    case 1:
      return R == 4 ? (StreamKernel)stream_gemv_kernel<F, 4, 1> : R == 2 ? (StreamKernel)stream_gemv_kernel<F, 2, 1>
                                                                         : (StreamKernel)stream_gemv_kernel<F, 1, 1>;
    case 2:
      return R == 4 ? (StreamKernel)stream_gemv_kernel<F, 4, 2> : R == 2 ? (StreamKernel)stream_gemv_kernel<F, 2, 2>
                                                                         : (StreamKernel)stream_gemv_kernel<F, 1, 2>;
    case 4:
      return R >= 2 ? (StreamKernel)stream_gemv_kernel<F, 2, 4> : (StreamKernel)stream_gemv_kernel<F, 1, 4>;
    default:
      return R >= 2 ? (StreamKernel)stream_gemv_kernel<F, 2, 8> : (StreamKernel)stream_gemv_kernel<F, 1, 8>;
  }
}

// Runs x [batch,in] through the streaming kernel in batch tiles that fit shared memory.
// Returns GOPH_E_UNSUPPORTED when even one activation row does not fit.
template <class F>
static int stream_launch(StreamArgs a, int device, int batch, cudaStream_t stream, int force_rows = 0) {
  DeviceState& st = device_state(device);
  a.iters = (a.units + 31) / 32;
  if (stream_smem_bytes<F>(1, a.iters) > (size_t)kSmemBudget)
    return fail(GOPH_E_UNSUPPORTED, "in_dim=%d: one activation row does not fit in shared memory", a.in_dim);
  int tile = 8;
  while (tile > 1 && stream_smem_bytes<F>(tile, a.iters) > (size_t)kSmemBudget) tile >>= 1;
  const float* x0 = a.x;
  float* out0 = a.out;
  for (int b0 = 0; b0 < batch; b0 += tile) {
    int nb = batch - b0 < tile ? batch - b0 : tile;
    int M = nb <= 1 ? 1 : nb <= 2 ? 2 : nb <= 4 ? 4 : 8;
    int R = force_rows;
    if (R != 1 && R != 2 && R != 4) {
      long want = (long)st.sm_count * 2 * kGWarps * 2;
      R = a.rows / 4 >= want ? 4 : a.rows / 2 >= want ? 2 : 1;
    }
    if (M >= 4 && R == 4) R = 2;
    a.x = x0 + (size_t)b0 * a.in_dim;
    a.out = out0 + (size_t)b0 * a.rows;
    a.batch = nb;
    a.x_aligned = ((uintptr_t)a.x % 16) == 0;
    StreamKernel k = stream_pick<F>(R, M);
    size_t smem = stream_smem_bytes<F>(M, a.iters);
    GOPH_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    GOPH_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, kGThreads, smem));
    if (per_sm < 1) return fail(GOPH_E_UNSUPPORTED, "streaming kernel does not fit (smem %zu)", smem);
    int tasks = (a.rows + R - 1) / R;
    int grid = (tasks + kGWarps - 1) / kGWarps;
    if (grid > st.sm_count * per_sm) grid = st.sm_count * per_sm;
    note_launch();
    k<<<grid, kGThreads, smem, stream>>>(a);
    GOPH_CUDA(cudaGetLastError());
  }
  return GOPH_OK;
}

}  // namespace goph
