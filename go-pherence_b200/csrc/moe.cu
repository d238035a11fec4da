// Mixture-of-experts selected-expert projection on MLX 4-bit experts.
//
// Replaces the per-expert launch loop of model.moeForwardGPU (model/moe_gpu.go:49-303: router
// GEMV, D2H of the logits, host softmax/top-k, then for every selected expert three GEMV launches,
// SiLU-mul and a scaled accumulate) and the persistent-candidate kernel of
// MLXSelectedExpertPersistentCandidate.Run (backends/nvidia/runtime/mlx_selected_expert.go:77-177).
// Arithmetic specification: moeForwardWithREAP (model/moe.go:203-347):
//   p = softmax(router . x) over all experts (exp taken in f64, sum in order), top-k by repeated
//   strict-'>' argmax, optional renormalisation; for every selected expert in selection order
//   h = silu(gate . x) * (up . x), d = down . h, out += weight * d.
//
// Five launches per call, whatever the number of tokens; nothing returns to the host:
//   1. router logits     — the MLX GEMV/GEMM kernel (batch = tokens)
//   2. moe_route_kernel  — one warp per token does the softmax/top-k in the reference's order; the
//      last CTA to finish then groups the (token, slot) items by expert: the list of experts that
//      were selected at all and, per expert, its items in (token, slot) order
//   3. moe_gate_up_kernel — grid (row blocks, selected experts): a warp streams row r of the
//      expert's gate and up matrices ONCE and applies it to up to four of the expert's tokens at a
//      time (their x staged in shared memory), writing silu(g) * u per item
//   4. moe_down_kernel   — same grouping for the down matrices, writing one vector per item
//   5. moe_combine_kernel — out[t] = sum over the token's slots, in selection order, of
//      weight * vector, so the result does not depend on scheduling.
// Each expert matrix is read from HBM once per call however many tokens chose the expert.
// Experts that are not resident on this GPU (multi-GPU placement) are skipped: the output is then
// this GPU's partial sum.
#include <string.h>

#include "goph_internal.cuh"

namespace goph {

constexpr uint32_t kMagicMoE = 0x4d4f4558;  // "MOEX"
constexpr int kMoeWarps = 8, kMoeThreads = kMoeWarps * 32;

struct MoeTables {
  const uint4** gate_w;   // [E] packed rows (16-byte units) or null when the expert is not resident
  const void** gate_sb;   // [E] {scale,bias} table
  const uint4** up_w;
  const void** up_sb;
  const uint4** down_w;
  const void** down_sb;
};

}  // namespace goph

struct goph_moe_layer {
  uint32_t magic;
  int device;
  int num_experts, hidden, inter, top_k, norm_topk, max_tokens, group_size;
  int sb_bf16;                     // all experts share the table type
  const goph_mlx_weight* router;   // borrowed
  goph::MoeTables host, dev;       // pointer tables (host mirror, device copy)
  int tables_dirty;
  float* logits;                   // [max_tokens][E]
  int* ids;                        // [max_tokens][top_k], -1 = none
  float* wts;                      // [max_tokens][top_k]
  float* act;                      // [max_tokens][top_k][inter]
  float* dpart;                    // [max_tokens][top_k][hidden] per-item down projections
  int* lists;                      // [0] arrival counter, [1] number of selected resident experts,
                                   // [2..2+E) their ids, [2+E..2+2E) items per expert,
                                   // [2+2E..) items [E][max_tokens]
};

namespace goph {

// nibble -> 16 + n by bit placement (top mantissa bits under 2^4)
__device__ __forceinline__ void unpack16(uint32_t w, float (&f)[8]) {
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

// Stages n floats (n a multiple of 32) as [iteration][slot][lane] float4 plus per-unit {16*sum, sum}.
// No barrier inside: the caller synchronises after staging all vectors.
__device__ __forceinline__ void moe_stage_values(const float* __restrict__ x, int n, float4* xs) {
  const int units = n / 32, iters = (units + 31) / 32;
  for (int idx = threadIdx.x; idx < iters * 256; idx += kMoeThreads) {
    int it = idx >> 8, slot = (idx >> 5) & 7, l = idx & 31, unit = it * 32 + l;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (unit < units) v = *reinterpret_cast<const float4*>(x + (size_t)unit * 32 + slot * 4);
    xs[idx] = v;
  }
}
__device__ __forceinline__ void moe_stage_consts(int n, const float4* xs, float2* xc) {
  const int units = n / 32, iters = (units + 31) / 32;
  for (int idx = threadIdx.x; idx < iters * 32; idx += kMoeThreads) {
    int it = idx >> 5, l = idx & 31;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float4 v = xs[(it * 8 + k) * 32 + l];
      s += (v.x + v.y) + (v.z + v.w);
    }
    xc[idx] = make_float2(16.f * s, s);
  }
}

struct MoeRow {
  const uint4* w;
  const void* sb;
};

// NW rows (of NW matrices, all `units` 16-byte units wide) against M staged vectors: acc[w][m] gets
// the per-lane partial of row w . vector m.  Each packed word is unpacked once and used M times.
template <bool SB_BF16, int NW, int M>
__device__ __forceinline__ void moe_rows_dot(const MoeRow (&rows)[NW], int units, int ug_shift, const float4* xs,
                                             const float2* xc, int xs_stride, int xc_stride, int lane,
                                             float (&acc)[NW][M]) {
  const int iters = (units + 31) / 32;
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[w][m] = 0.f;
  for (int it = 0; it < iters; ++it) {
    int unit = it * 32 + lane;
    const bool valid = unit < units;
    if (!valid) unit = units - 1;
    uint4 q[NW];
    float sc[NW], bi[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) q[w] = ld_stream(rows[w].w + unit);
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      if (SB_BF16) {
        uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(rows[w].sb) + (unit >> ug_shift));
        sc[w] = __uint_as_float(v << 16);
        bi[w] = __uint_as_float(v & 0xFFFF0000u);
      } else {
        float2 v = __ldg(reinterpret_cast<const float2*>(rows[w].sb) + (unit >> ug_shift));
        sc[w] = v.x;
        bi[w] = v.y;
      }
    }
    float2 F[NW][M];
#pragma unroll
    for (int w = 0; w < NW; ++w)
#pragma unroll
      for (int m = 0; m < M; ++m) F[w][m] = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float f[NW][8];
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const uint32_t word = k == 0 ? q[w].x : k == 1 ? q[w].y : k == 2 ? q[w].z : q[w].w;
        unpack16(word, f[w]);
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float4 xa = xs[m * xs_stride + (it * 8 + 2 * k) * 32 + lane];
        float4 xb = xs[m * xs_stride + (it * 8 + 2 * k + 1) * 32 + lane];
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          fma2(F[w][m], make_float2(f[w][0], f[w][1]), make_float2(xa.x, xa.y));
          fma2(F[w][m], make_float2(f[w][2], f[w][3]), make_float2(xa.z, xa.w));
          fma2(F[w][m], make_float2(f[w][4], f[w][5]), make_float2(xb.x, xb.y));
          fma2(F[w][m], make_float2(f[w][6], f[w][7]), make_float2(xb.z, xb.w));
        }
      }
    }
    if (valid) {
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float2 c = xc[m * xc_stride + it * 32 + lane];
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          acc[w][m] = fmaf(sc[w], (F[w][m].x + F[w][m].y) - c.x, acc[w][m]);
          acc[w][m] = fmaf(bi[w], c.y, acc[w][m]);
        }
      }
    }
  }
}

__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// simd.SoftmaxInPlace + the top-k loop of moeForwardWithREAP in the reference's order
// (model/moe.go:226-280; backends/simd/runtime/softmax.go:9-30): one CTA per token; the
// exponentials are taken in parallel, the sum by one thread in index order, the k rounds of
// "largest probability not yet picked, lowest id on ties" by a warp.  The last CTA to finish groups
// the items by expert.
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int num_experts, int top_k, int norm_topk, int tokens,
                 int max_tokens, MoeTables tb, int* __restrict__ ids, float* __restrict__ wts,
                 float* __restrict__ probs_scratch, int* __restrict__ lists) {
  pdl_prologue();
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
  const float* lg = logits + (size_t)t * num_experts;
  float* p = probs_scratch + (size_t)t * num_experts;
  int* my_ids = ids + (size_t)t * top_k;
  float* my_w = wts + (size_t)t * top_k;
  __shared__ float s_mx, s_inv;
  __shared__ int s_ok, s_last;
  if (tid < 32) {
    float mx = -INFINITY;
    for (int i = lane; i < num_experts; i += 32) mx = fmaxf(mx, lg[i]);  // skips NaN, as "x > mx" does
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // the reference starts from x[0]: if that is NaN every comparison is false and the maximum stays NaN
    if (isnan(lg[0])) mx = lg[0];
    if (lane == 0) s_mx = mx;
  }
  __syncthreads();
  for (int i = tid; i < num_experts; i += blockDim.x) p[i] = (float)exp((double)(lg[i] - s_mx));
  __syncthreads();
  if (tid == 0) {
    float sum = 0.f;
    for (int i = 0; i < num_experts; ++i) sum = __fadd_rn(sum, p[i]);
    s_ok = !(sum == 0.f || isnan(sum) || isinf(sum));  // SoftmaxInPlace fails: no expert runs
    s_inv = __fdiv_rn(1.f, sum);
  }
  __syncthreads();
  if (s_ok)
    for (int i = tid; i < num_experts; i += blockDim.x) p[i] = __fmul_rn(p[i], s_inv);
  __syncthreads();
  if (tid < 32) {
    int n = 0;
    float wsum = 0.f;
    for (int k = 0; k < top_k; ++k) {
      int best = -1;
      float bs = -1.f;
      if (s_ok) {
        for (int j = lane; j < num_experts; j += 32) {
          float v = p[j];
          if (v > bs) {
            bool picked = false;
            for (int q = 0; q < n; ++q) picked |= my_ids[q] == j;
            if (!picked) {
              best = j;
              bs = v;
            }
          }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          float ov = __shfl_xor_sync(0xffffffffu, bs, o);
          int oi = __shfl_xor_sync(0xffffffffu, best, o);
          if (oi >= 0 && (best < 0 || ov > bs || (ov == bs && oi < best))) {
            bs = ov;
            best = oi;
          }
        }
      }
      if (best >= 0) {
        if (lane == 0) {
          my_ids[n] = best;
          my_w[n] = bs;
        }
        wsum = __fadd_rn(wsum, bs);
        ++n;
      }
      __syncwarp();
    }
    if (lane == 0) {
      for (int k = n; k < top_k; ++k) {
        my_ids[k] = -1;
        my_w[k] = 0.f;
      }
      if (norm_topk && n > 0 && wsum > 0.f)
        for (int k = 0; k < n; ++k) my_w[k] = __fdiv_rn(my_w[k], wsum);
      __threadfence();
      s_last = atomicAdd(&lists[0], 1) == tokens - 1;
    }
  }
  __syncthreads();
  if (!s_last) return;
  // ---- last CTA: group the items by expert ------------------------------------------------
  __threadfence();
  int* n_active = lists + 1;
  int* active = lists + 2;
  int* counts = lists + 2 + num_experts;
  int* items = lists + 2 + 2 * num_experts;
  const volatile int* vids = ids;
  for (int e = tid; e < num_experts; e += blockDim.x) {
    int c = 0;
    if (tb.gate_w[e] != nullptr)
      for (int it = 0; it < tokens * top_k; ++it)
        if (vids[it] == e) items[(size_t)e * max_tokens + c++] = it;  // a token selects an expert at most once
    counts[e] = c;
  }
  __syncthreads();
  if (tid == 0) {
    int n = 0;
    for (int e = 0; e < num_experts; ++e)
      if (counts[e] > 0) active[n++] = e;
    *n_active = n;
    lists[0] = 0;  // ready for the next call
  }
}

constexpr int kMoeM = 4;  // tokens of one expert handled per pass over its rows

// act[item][r] = silu(gate_e[r] . x_t) * (up_e[r] . x_t) for every item (token t, slot) of expert e.
template <bool SB_BF16>
__global__ void __launch_bounds__(kMoeThreads)
moe_gate_up_kernel(MoeTables tb, const float* __restrict__ x, const int* __restrict__ lists, float* __restrict__ act,
                   int num_experts, int max_tokens, int hidden, int inter, int top_k, int ug_shift, int groups) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_prologue();
  if ((int)blockIdx.y >= lists[1]) return;
  const int e = lists[2 + blockIdx.y];
  const int count = lists[2 + num_experts + e];
  const int* items = lists + 2 + 2 * num_experts + (size_t)e * max_tokens;
  const int units = hidden / 32, iters = (units + 31) / 32;
  const int xs_stride = iters * 256, xc_stride = iters * 32;
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)kMoeM * xs_stride * 16);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t sb_row = (size_t)groups * (SB_BF16 ? 4 : 8);
  for (int base = 0; base < count; base += kMoeM) {
    const int m_now = min(kMoeM, count - base);
    if (base) __syncthreads();
    for (int m = 0; m < m_now; ++m) moe_stage_values(x + (size_t)(items[base + m] / top_k) * hidden, hidden, xs + m * xs_stride);
    __syncthreads();
    for (int m = 0; m < m_now; ++m) moe_stage_consts(hidden, xs + m * xs_stride, xc + m * xc_stride);
    __syncthreads();
    for (int r = blockIdx.x * kMoeWarps + warp; r < inter; r += gridDim.x * kMoeWarps) {
      const MoeRow rows[2] = {{tb.gate_w[e] + (size_t)r * units, reinterpret_cast<const char*>(tb.gate_sb[e]) + r * sb_row},
                              {tb.up_w[e] + (size_t)r * units, reinterpret_cast<const char*>(tb.up_sb[e]) + r * sb_row}};
      float g[kMoeM], u[kMoeM];
      if (m_now == 1) {
        float acc[2][1];
        moe_rows_dot<SB_BF16, 2, 1>(rows, units, ug_shift, xs, xc, xs_stride, xc_stride, lane, acc);
        g[0] = acc[0][0];
        u[0] = acc[1][0];
      } else {
        float acc[2][kMoeM];  // vectors past m_now are stale shared memory; their results are not stored
        moe_rows_dot<SB_BF16, 2, kMoeM>(rows, units, ug_shift, xs, xc, xs_stride, xc_stride, lane, acc);
#pragma unroll
        for (int m = 0; m < kMoeM; ++m) {
          g[m] = acc[0][m];
          u[m] = acc[1][m];
        }
      }
#pragma unroll
      for (int m = 0; m < kMoeM; ++m) {
        if (m < m_now) {
          float gs = warp_sum(g[m]), us = warp_sum(u[m]);
          if (lane == 0) {
            // kernels.SiLU then the multiply (backends/simd/kernels/activation.go:15-24)
            float sv = __fdiv_rn(gs, __fadd_rn(1.0f, (float)exp((double)(-gs))));
            act[(size_t)items[base + m] * inter + r] = __fmul_rn(sv, us);
          }
        }
      }
    }
  }
}

// dpart[item][r] = down_e[r] . act[item] for every item of expert e.
template <bool SB_BF16>
__global__ void __launch_bounds__(kMoeThreads)
moe_down_kernel(MoeTables tb, const float* __restrict__ act, const int* __restrict__ lists, float* __restrict__ dpart,
                int num_experts, int max_tokens, int hidden, int inter, int ug_shift, int groups) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_prologue();
  if ((int)blockIdx.y >= lists[1]) return;
  const int e = lists[2 + blockIdx.y];
  const int count = lists[2 + num_experts + e];
  const int* items = lists + 2 + 2 * num_experts + (size_t)e * max_tokens;
  const int units = inter / 32, iters = (units + 31) / 32;
  const int xs_stride = iters * 256, xc_stride = iters * 32;
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)kMoeM * xs_stride * 16);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t sb_row = (size_t)groups * (SB_BF16 ? 4 : 8);
  for (int base = 0; base < count; base += kMoeM) {
    const int m_now = min(kMoeM, count - base);
    if (base) __syncthreads();
    for (int m = 0; m < m_now; ++m) moe_stage_values(act + (size_t)items[base + m] * inter, inter, xs + m * xs_stride);
    __syncthreads();
    for (int m = 0; m < m_now; ++m) moe_stage_consts(inter, xs + m * xs_stride, xc + m * xc_stride);
    __syncthreads();
    // two rows per pass: the rows are short, two loads in flight per lane
    for (int r = (blockIdx.x * kMoeWarps + warp) * 2; r < hidden; r += gridDim.x * kMoeWarps * 2) {
      const int r1 = min(r + 1, hidden - 1);
      const MoeRow rows[2] = {{tb.down_w[e] + (size_t)r * units, reinterpret_cast<const char*>(tb.down_sb[e]) + r * sb_row},
                              {tb.down_w[e] + (size_t)r1 * units, reinterpret_cast<const char*>(tb.down_sb[e]) + r1 * sb_row}};
      float d0[kMoeM], d1[kMoeM];
      if (m_now == 1) {
        float acc[2][1];
        moe_rows_dot<SB_BF16, 2, 1>(rows, units, ug_shift, xs, xc, xs_stride, xc_stride, lane, acc);
        d0[0] = acc[0][0];
        d1[0] = acc[1][0];
      } else {
        float acc[2][kMoeM];
        moe_rows_dot<SB_BF16, 2, kMoeM>(rows, units, ug_shift, xs, xc, xs_stride, xc_stride, lane, acc);
#pragma unroll
        for (int m = 0; m < kMoeM; ++m) {
          d0[m] = acc[0][m];
          d1[m] = acc[1][m];
        }
      }
#pragma unroll
      for (int m = 0; m < kMoeM; ++m) {
        if (m < m_now) {
          float a0 = warp_sum(d0[m]), a1 = warp_sum(d1[m]);
          if (lane == 0) {
            float* o = dpart + (size_t)items[base + m] * hidden;
            o[r] = a0;
            if (r + 1 < hidden) o[r + 1] = a1;
          }
        }
      }
    }
  }
}

// out[t][r] = sum over slots k in selection order of weight[t][k] * dpart[t][k][r]
// (out[i] += weight * down[i], model/moe.go:336-344).  Slots whose expert is not resident here add nothing.
__global__ void __launch_bounds__(256)
moe_combine_kernel(MoeTables tb, const float* __restrict__ dpart, const int* __restrict__ ids,
                   const float* __restrict__ wts, float* __restrict__ out, int hidden, int top_k) {
  pdl_prologue();
  const int t = blockIdx.y;
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= hidden) return;
  float acc = 0.f;
  for (int k = 0; k < top_k; ++k) {
    const int e = ids[t * top_k + k];
    if (e < 0 || tb.down_w[e] == nullptr) continue;
    acc = __fadd_rn(acc, __fmul_rn(wts[t * top_k + k], dpart[((size_t)t * top_k + k) * hidden + r]));
  }
  out[(size_t)t * hidden + r] = acc;
}

template <typename... KArgs, typename... Args>
static int moe_launch(void (*k)(KArgs...), dim3 grid, int threads, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, k, KArgs(args)...));
  return GOPH_OK;
}

static bool valid_moe(const goph_moe_layer* m) { return m && m->magic == kMagicMoE; }

static int moe_upload_tables(goph_moe_layer* m) {
  if (!m->tables_dirty) return GOPH_OK;
  size_t n = (size_t)m->num_experts * sizeof(void*);
  GOPH_CUDA(cudaMemcpy((void*)m->dev.gate_w, m->host.gate_w, n, cudaMemcpyHostToDevice));
  GOPH_CUDA(cudaMemcpy((void*)m->dev.gate_sb, m->host.gate_sb, n, cudaMemcpyHostToDevice));
  GOPH_CUDA(cudaMemcpy((void*)m->dev.up_w, m->host.up_w, n, cudaMemcpyHostToDevice));
  GOPH_CUDA(cudaMemcpy((void*)m->dev.up_sb, m->host.up_sb, n, cudaMemcpyHostToDevice));
  GOPH_CUDA(cudaMemcpy((void*)m->dev.down_w, m->host.down_w, n, cudaMemcpyHostToDevice));
  GOPH_CUDA(cudaMemcpy((void*)m->dev.down_sb, m->host.down_sb, n, cudaMemcpyHostToDevice));
  m->tables_dirty = 0;
  return GOPH_OK;
}

}  // namespace goph

using namespace goph;

GOPH_API int goph_moe_create(int device, int num_experts, int hidden, int inter, int group_size, int top_k,
                             int norm_topk, int max_tokens, goph_moe_layer** out) {
  clear_error();
  if (!out) return fail(GOPH_E_INVALID, "goph_moe_create: nil result pointer");
  *out = nullptr;
  if (num_experts <= 0 || hidden <= 0 || inter <= 0 || max_tokens <= 0)
    return fail(GOPH_E_INVALID, "invalid MoE dims experts=%d hidden=%d inter=%d tokens=%d", num_experts, hidden, inter, max_tokens);
  if (top_k <= 0) top_k = 8;                      // model/moe.go:209-212
  if (top_k > num_experts) top_k = num_experts;   // model/moe.go:213-215
  if (group_size < 32 || (group_size & (group_size - 1)) || hidden % group_size || inter % group_size || hidden % 32 || inter % 32)
    return fail(GOPH_E_UNSUPPORTED, "MoE experts need a power-of-two group size >= 32 dividing hidden=%d and inter=%d", hidden, inter);
  if (int rc = use_device(device)) return rc;
  goph_moe_layer* m = new goph_moe_layer();
  memset(m, 0, sizeof *m);
  m->magic = kMagicMoE;
  m->device = device;
  m->num_experts = num_experts;
  m->hidden = hidden;
  m->inter = inter;
  m->top_k = top_k;
  m->norm_topk = norm_topk;
  m->max_tokens = max_tokens;
  m->group_size = group_size;
  m->sb_bf16 = -1;
  size_t n = (size_t)num_experts;
  const void*** hp[6] = {(const void***)&m->host.gate_w, &m->host.gate_sb, (const void***)&m->host.up_w,
                         &m->host.up_sb,                 (const void***)&m->host.down_w, &m->host.down_sb};
  const void*** dp[6] = {(const void***)&m->dev.gate_w, &m->dev.gate_sb, (const void***)&m->dev.up_w,
                         &m->dev.up_sb,                 (const void***)&m->dev.down_w, &m->dev.down_sb};
  cudaError_t e = cudaSuccess;
  for (int i = 0; i < 6 && e == cudaSuccess; ++i) {
    *hp[i] = new const void*[n]();
    e = cudaMalloc((void**)dp[i], n * sizeof(void*));
  }
  if (e == cudaSuccess) e = cudaMalloc(&m->logits, (size_t)max_tokens * num_experts * 2 * sizeof(float));  // logits + probabilities
  if (e == cudaSuccess) e = cudaMalloc(&m->ids, (size_t)max_tokens * top_k * sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(&m->wts, (size_t)max_tokens * top_k * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&m->act, (size_t)max_tokens * top_k * inter * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&m->dpart, (size_t)max_tokens * top_k * hidden * sizeof(float));
  const size_t list_ints = 2 + 2 * (size_t)num_experts + (size_t)num_experts * max_tokens;
  if (e == cudaSuccess) e = cudaMalloc(&m->lists, list_ints * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(m->lists, 0, list_ints * sizeof(int));
  if (e != cudaSuccess) {
    int rc = fail_cuda(e, "cudaMalloc(MoE layer)");
    m->magic = 0;  // partial allocations are released by the process; the handle is not returned
    return rc;
  }
  m->tables_dirty = 1;
  *out = m;
  return GOPH_OK;
}

GOPH_API int goph_moe_set_router(goph_moe_layer* m, const goph_mlx_weight* router) {
  clear_error();
  if (!valid_moe(m)) return fail(GOPH_E_INVALID, "invalid MoE layer handle");
  if (router && (router->magic != kMagicMLX || router->in_dim != m->hidden || router->out_dim != m->num_experts))
    return fail(GOPH_E_INVALID, "router must be an MLX weight [%d x %d]", m->num_experts, m->hidden);
  m->router = router;
  return GOPH_OK;
}

GOPH_API int goph_moe_set_expert(goph_moe_layer* m, int eid, const goph_mlx_weight* gate, const goph_mlx_weight* up,
                                 const goph_mlx_weight* down) {
  clear_error();
  if (!valid_moe(m)) return fail(GOPH_E_INVALID, "invalid MoE layer handle");
  if (eid < 0 || eid >= m->num_experts) return fail(GOPH_E_INVALID, "expert id %d out of 0..%d", eid, m->num_experts - 1);
  if (!gate && !up && !down) {  // expert not resident on this GPU
    m->host.gate_w[eid] = m->host.up_w[eid] = m->host.down_w[eid] = nullptr;
    m->tables_dirty = 1;
    return GOPH_OK;
  }
  const goph_mlx_weight* ws[3] = {gate, up, down};
  const int want_out[3] = {m->inter, m->inter, m->hidden}, want_in[3] = {m->hidden, m->hidden, m->inter};
  for (int i = 0; i < 3; ++i) {
    const goph_mlx_weight* w = ws[i];
    if (!w || w->magic != kMagicMLX || w->device != m->device || w->out_dim != want_out[i] || w->in_dim != want_in[i] ||
        w->group_size != m->group_size)
      return fail(GOPH_E_INVALID, "expert %d: projection %d must be an MLX weight [%d x %d] with group size %d on device %d", eid, i,
                  want_out[i], want_in[i], m->group_size, m->device);
    if (!w->qweight || !w->sb)
      return fail(GOPH_E_UNSUPPORTED, "expert %d: projection %d is in the tiled layout; experts use the row-major layout", eid, i);
    if (m->sb_bf16 >= 0 && m->sb_bf16 != w->sb_bf16)
      return fail(GOPH_E_UNSUPPORTED, "experts mix bf16-valued and f32 scale tables");
    m->sb_bf16 = w->sb_bf16;
  }
  m->host.gate_w[eid] = reinterpret_cast<const uint4*>(gate->qweight);
  m->host.gate_sb[eid] = gate->sb;
  m->host.up_w[eid] = reinterpret_cast<const uint4*>(up->qweight);
  m->host.up_sb[eid] = up->sb;
  m->host.down_w[eid] = reinterpret_cast<const uint4*>(down->qweight);
  m->host.down_sb[eid] = down->sb;
  m->tables_dirty = 1;
  return GOPH_OK;
}

GOPH_API int goph_moe_free(goph_moe_layer* m) {
  clear_error();
  if (!m) return GOPH_OK;
  if (!valid_moe(m)) return fail(GOPH_E_INVALID, "goph_moe_free: not a MoE layer handle");
  if (int rc = use_device(m->device)) return rc;
  const void** hp[6] = {(const void**)m->host.gate_w, m->host.gate_sb, (const void**)m->host.up_w,
                        m->host.up_sb,                (const void**)m->host.down_w, m->host.down_sb};
  const void** dp[6] = {(const void**)m->dev.gate_w, m->dev.gate_sb, (const void**)m->dev.up_w,
                        m->dev.up_sb,                (const void**)m->dev.down_w, m->dev.down_sb};
  for (int i = 0; i < 6; ++i) {
    delete[] hp[i];
    cudaFree((void*)dp[i]);
  }
  cudaFree(m->logits);
  cudaFree(m->ids);
  cudaFree(m->wts);
  cudaFree(m->act);
  cudaFree(m->dpart);
  cudaFree(m->lists);
  m->magic = 0;
  delete m;
  return GOPH_OK;
}

// Launches 2-5 for routing given as logits already on the device.
static int moe_run(goph_moe_layer* m, float* out_dev, const float* x_dev, const float* logits_dev, int tokens,
                   cudaStream_t s) {
  if (int rc = moe_upload_tables(m)) return rc;
  const int sms = device_state(m->device).sm_count;
  float* probs = m->logits + (size_t)m->max_tokens * m->num_experts;
  if (int rc = moe_launch(moe_route_kernel, dim3(tokens), 128, 0, s, logits_dev, m->num_experts, m->top_k, m->norm_topk, tokens,
                          m->max_tokens, m->dev, m->ids, m->wts, probs, m->lists))
    return rc;
  int sh = 0;
  while ((32 << sh) < m->group_size) ++sh;
  // at most this many experts can have been selected; CTAs past the actual number return at once
  const int max_active = min(m->num_experts, tokens * m->top_k);
  const int want_ctas = sms * 8;
  {
    const int units = m->hidden / 32, iters = (units + 31) / 32;
    const size_t smem = (size_t)kMoeM * iters * (256 * 16 + 32 * 8);
    if (smem > (size_t)kSmemBudget) return fail(GOPH_E_UNSUPPORTED, "MoE: hidden=%d does not fit shared memory", m->hidden);
    const int max_blocks = (m->inter + kMoeWarps - 1) / kMoeWarps;
    int gx = max(1, min(max_blocks, (want_ctas + max_active - 1) / max_active));
    auto k = m->sb_bf16 ? moe_gate_up_kernel<true> : moe_gate_up_kernel<false>;
    GOPH_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (int rc = moe_launch(k, dim3(gx, max_active), kMoeThreads, smem, s, m->dev, x_dev, m->lists, m->act, m->num_experts,
                            m->max_tokens, m->hidden, m->inter, m->top_k, sh, m->hidden / m->group_size))
      return rc;
  }
  {
    const int units = m->inter / 32, iters = (units + 31) / 32;
    const size_t smem = (size_t)kMoeM * iters * (256 * 16 + 32 * 8);
    if (smem > (size_t)kSmemBudget) return fail(GOPH_E_UNSUPPORTED, "MoE: inter=%d does not fit shared memory", m->inter);
    const int max_blocks = (m->hidden + kMoeWarps * 2 - 1) / (kMoeWarps * 2);
    int gx = max(1, min(max_blocks, (want_ctas + max_active - 1) / max_active));
    auto k = m->sb_bf16 ? moe_down_kernel<true> : moe_down_kernel<false>;
    GOPH_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (int rc = moe_launch(k, dim3(gx, max_active), kMoeThreads, smem, s, m->dev, m->act, m->lists, m->dpart, m->num_experts,
                            m->max_tokens, m->hidden, m->inter, sh, m->inter / m->group_size))
      return rc;
  }
  return moe_launch(moe_combine_kernel, dim3((m->hidden + 255) / 256, tokens), 256, 0, s, m->dev, m->dpart, m->ids, m->wts,
                    out_dev, m->hidden, m->top_k);
}

static int moe_check_io(const goph_moe_layer* m, const float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                        int tokens) {
  if (!valid_moe(m)) return fail(GOPH_E_INVALID, "invalid MoE layer handle");
  if (tokens <= 0 || tokens > m->max_tokens) return fail(GOPH_E_INVALID, "tokens=%d not in 1..%d", tokens, m->max_tokens);
  uint64_t need = (uint64_t)tokens * m->hidden;
  if (!x_dev || x_len < need || !out_dev || out_len < need)
    return fail(GOPH_E_INVALID, "MoE buffers x=%llu out=%llu, want at least %llu", (unsigned long long)x_len,
                (unsigned long long)out_len, (unsigned long long)need);
  if ((uintptr_t)x_dev % 16) return fail(GOPH_E_INVALID, "MoE x must be 16-byte aligned");
  if (m->sb_bf16 < 0) return fail(GOPH_E_INVALID, "MoE layer has no resident expert");
  return GOPH_OK;
}

GOPH_API int goph_moe_forward(goph_moe_layer* m, float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                              int tokens, void* stream) {
  clear_error();
  if (int rc = moe_check_io(m, out_dev, out_len, x_dev, x_len, tokens)) return rc;
  if (!m->router) return fail(GOPH_E_INVALID, "MoE layer has no router weight");
  if (int rc = use_device(m->device)) return rc;
  if (int rc = goph_mlx_gemm(m->logits, (uint64_t)tokens * m->num_experts, x_dev, x_len, m->router, tokens, stream)) return rc;
  return moe_run(m, out_dev, x_dev, m->logits, tokens, (cudaStream_t)stream);
}

GOPH_API int goph_moe_forward_logits(goph_moe_layer* m, float* out_dev, uint64_t out_len, const float* x_dev,
                                     uint64_t x_len, const float* logits_dev, uint64_t logits_len, int tokens,
                                     void* stream) {
  clear_error();
  if (int rc = moe_check_io(m, out_dev, out_len, x_dev, x_len, tokens)) return rc;
  if (!logits_dev || logits_len < (uint64_t)tokens * m->num_experts) return fail(GOPH_E_INVALID, "router logits buffer too short");
  if (int rc = use_device(m->device)) return rc;
  return moe_run(m, out_dev, x_dev, logits_dev, tokens, (cudaStream_t)stream);
}

GOPH_API int goph_moe_last_routing(goph_moe_layer* m, int tokens, int* ids_host, float* weights_host) {
  clear_error();
  if (!valid_moe(m)) return fail(GOPH_E_INVALID, "invalid MoE layer handle");
  if (tokens <= 0 || tokens > m->max_tokens || !ids_host || !weights_host) return fail(GOPH_E_INVALID, "bad routing query");
  if (int rc = use_device(m->device)) return rc;
  GOPH_CUDA(cudaMemcpy(ids_host, m->ids, (size_t)tokens * m->top_k * sizeof(int), cudaMemcpyDeviceToHost));
  GOPH_CUDA(cudaMemcpy(weights_host, m->wts, (size_t)tokens * m->top_k * sizeof(float), cudaMemcpyDeviceToHost));
  return GOPH_OK;
}
