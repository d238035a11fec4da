// GGUF products addressed by a work list, for MoE layers whose experts are stacked in one matrix:
//   * gate/up with the activation fused: out[w][i] = gelu_tanh(gate_i . x_w) * (up_i . x_w), the
//     rows of expert work_experts[w] (nvidia.GateUpGELUQ4KBatchToBuffer / GateUpGELUQ4KByWorkToBuffer,
//     backends/nvidia/runtime/q4k.go:322-352; kernel text backends/nvidia/ptx/q4/gate_up_gelu_q4k*.go);
//   * down projection with a weighted scatter-add: dst[pos[w]][r] += weight[w] * (W_e[r] . x_w)
//     (nvidia.GemvQ8_0BatchScatter / GemvQ8_0ScatterByWork, backends/nvidia/runtime/q8.go:193-222;
//     kernel text backends/nvidia/ptx/q8/q8_scatter*.go).
// Both for Q4_K and Q8_0 matrices in either device layout (the reference has the first for Q4_K and
// the second for Q8_0 only).  CUDA-core kernels: one warp per (output row, work item), a lane takes
// 32-element units of the row; the weights of an item's expert are read once per item.  The indices
// of a work list live in device memory, so the kernels check them: an expert index outside the
// matrix or a destination outside dst is skipped and recorded in the status word (601 / 602).
#include <string.h>

#include <mutex>

#include "goph_internal.cuh"
#include "gguf_fmt.cuh"

namespace goph {
namespace {

constexpr int kWarps = 8;
constexpr int kQ4KStage = 128 * 128 + 128 * 16;   // tensor-core layout: nibbles + headers of a stage
constexpr int kQ80Stage = 128 * 256 + 128 * 16;   // bytes + f16 scales

struct WorkView {
  const uint8_t* data;
  const uint16_t* d16;
  const uint8_t* tiled;
  int qtype, in_dim, out_dim, nchunks;
};

__device__ __forceinline__ float f16f(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)(h & 0xFFFFu))); }

// sum over the 32 elements of `unit` of row `row` of w_e * x_e, with the roundings of the
// dequantisation (sc*d and m*dmin, d*q) and f32 accumulation
__device__ __forceinline__ float unit_dot(const WorkView& v, int row, int unit, const float* __restrict__ x) {
  const float4* xp = reinterpret_cast<const float4*>(x + (size_t)unit * 32);
  float xs[32];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float4 t = __ldg(xp + k);
    xs[4 * k] = t.x; xs[4 * k + 1] = t.y; xs[4 * k + 2] = t.z; xs[4 * k + 3] = t.w;
  }
  const int chunk = unit >> 3, s = unit & 7, r = row & 127;
  if (v.qtype == GOPH_GGUF_Q4_K) {
    uint4 h, q;
    if (v.tiled) {
      const uint8_t* stg = v.tiled + ((size_t)(row >> 7) * v.nchunks + chunk) * kQ4KStage;
      h = *reinterpret_cast<const uint4*>(stg + 128 * 128 + r * 16);
      q = *reinterpret_cast<const uint4*>(stg + r * 128 + ((s ^ (r & 7)) << 4));
    } else {
      const uint8_t* blk = v.data + ((size_t)row * v.nchunks + chunk) * 144;
      h = *reinterpret_cast<const uint4*>(blk);
      q = *reinterpret_cast<const uint4*>(blk + 16 + 16 * s);
    }
    const int bit = 12 * s, wi = bit >> 5, sh = bit & 31;
    const uint32_t lo = wi == 0 ? h.y : wi == 1 ? h.z : h.w, hi = wi == 0 ? h.z : wi == 1 ? h.w : 0u;
    const uint32_t f = __funnelshift_r(lo, hi, sh) & 0xFFFu;
    const float sd = __fmul_rn((float)(f & 63u), f16f(h.x)), md = __fmul_rn((float)(f >> 6), f16f(h.x >> 16));
    const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc = fmaf(__fsub_rn(__fmul_rn(sd, (float)((ws[k] >> (4 * e)) & 0xFu)), md), xs[8 * k + e], acc);
    }
    return acc;
  }
  // Q8_0
  float d;
  uint4 b[2];
  bool biased;
  if (v.tiled) {
    const uint8_t* stg = v.tiled + ((size_t)(row >> 7) * v.nchunks + chunk) * kQ80Stage;
    const uint8_t* p = stg + s * 4096 + (r >> 3) * 128 + (r & 7) * 16;
    b[0] = *reinterpret_cast<const uint4*>(p);
    b[1] = *reinterpret_cast<const uint4*>(p + 2048);
    d = f16f(*reinterpret_cast<const uint16_t*>(stg + 128 * 256 + r * 16 + s * 2));
    biased = false;  // signed bytes
  } else {
    const uint8_t* p = v.data + (size_t)row * v.in_dim + (size_t)unit * 32;
    b[0] = *reinterpret_cast<const uint4*>(p);
    b[1] = *reinterpret_cast<const uint4*>(p + 16);
    d = f16f(v.d16[(size_t)row * (v.in_dim / 32) + unit]);
    biased = true;  // q + 128
  }
  float acc = 0.f;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const uint32_t ws[4] = {b[hh].x, b[hh].y, b[hh].z, b[hh].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int byte = (int)((ws[k] >> (8 * e)) & 0xFFu);
        const int q = biased ? byte - 128 : (int)(signed char)byte;
        acc = fmaf(__fmul_rn(d, (float)q), xs[16 * hh + 4 * k + e], acc);
      }
    }
  }
  return acc;
}

__device__ __forceinline__ float row_dot(const WorkView& v, int row, const float* __restrict__ x, int lane) {
  float acc = 0.f;
  for (int unit = lane; unit < v.in_dim / 32; unit += 32) acc += unit_dot(v, row, unit, x);
  return warp_sum(acc);
}

// GELU in the tanh form of the reference kernel: 0.5 g (1 + tanh(0.79788456 (g + 0.044715 g^3)))
__device__ __forceinline__ float gelu_tanh(float g) {
  const float u = 0.7978845608f * fmaf(0.044715f, g * g * g, g);
  const float t = 2.f / (1.f + __expf(-2.f * u)) - 1.f;
  return 0.5f * g * (1.f + t);
}

// grid (row blocks, items); a warp per (intermediate row i, item w)
__global__ void __launch_bounds__(kWarps * 32)
gate_up_gelu_kernel(WorkView v, const float* __restrict__ x, const uint32_t* __restrict__ work_experts, int active_experts,
                    int inter, float* __restrict__ out, int* __restrict__ status) {
  const int lane = threadIdx.x & 31, i = blockIdx.x * kWarps + (threadIdx.x >> 5), w = blockIdx.y;
  if (i >= inter) return;
  const uint32_t e = work_experts ? work_experts[w] : 0u;
  if (e >= (uint32_t)active_experts) {
    if (lane == 0) atomicCAS(status, 0, 601);
    return;
  }
  const float* xw = x + (size_t)w * v.in_dim;
  const int gate_row = (int)e * 2 * inter + i;
  const float g = row_dot(v, gate_row, xw, lane), u = row_dot(v, gate_row + inter, xw, lane);
  if (lane == 0) out[(size_t)w * inter + i] = gelu_tanh(g) * u;
}

// grid (row blocks, items); a warp per (expert row r, item w): dst[pos][r] += weight * (W_e[r] . x_w)
__global__ void __launch_bounds__(kWarps * 32)
scatter_by_work_kernel(WorkView v, const float* __restrict__ x, const uint32_t* __restrict__ work_active,
                       const uint32_t* __restrict__ work_pos, const float* __restrict__ work_weight, int active_experts,
                       int expert_out, float* __restrict__ dst, unsigned long long dst_len, int* __restrict__ status) {
  const int lane = threadIdx.x & 31, r = blockIdx.x * kWarps + (threadIdx.x >> 5), w = blockIdx.y;
  if (r >= expert_out) return;
  const uint32_t e = work_active ? work_active[w] : 0u;
  const unsigned long long at = (unsigned long long)work_pos[w] * (unsigned long long)expert_out + (unsigned long long)r;
  if (e >= (uint32_t)active_experts || at >= dst_len) {
    if (lane == 0) atomicCAS(status, 0, e >= (uint32_t)active_experts ? 601 : 602);
    return;
  }
  const float y = row_dot(v, (int)e * expert_out + r, x + (size_t)w * v.in_dim, lane);
  if (lane == 0) atomicAdd(dst + at, y * work_weight[w]);  // items may share a destination row
}

// The streaming policies reading the tensor-core layouts instead (one stage per 128 rows x 256
// elements, see mlx_mma.cu): the same 16 bytes per unit, found at the stage's addresses.  StreamArgs::w
// is the tiled buffer, row_bytes the number of 256-element chunks of a row.
struct Q4KTiledFmt : Q4KFmt {
  static __device__ __forceinline__ void load(const StreamArgs& a, int row, int unit, Row& t) {
    const int s = unit & 7, r = row & 127;
    const uint8_t* stg = a.w + ((size_t)(row >> 7) * a.row_bytes + (unit >> 3)) * kQ4KStage;
    const uint4 h = __ldg(reinterpret_cast<const uint4*>(stg + 128 * 128 + r * 16));
    t.q = ld_stream(reinterpret_cast<const uint4*>(stg + r * 128 + ((s ^ (r & 7)) << 4)));
    const uint32_t f = q4k_field(h, s);
    t.sd = __fmul_rn((float)(f & 63u), f16_bits_to_f32(h.x & 0xFFFFu));
    t.md = __fmul_rn((float)(f >> 6), f16_bits_to_f32(h.x >> 16));
  }
};
struct Q80TiledFmt : Q80Fmt {
  static __device__ __forceinline__ void load(const StreamArgs& a, int row, int unit, Row& t) {
    // unit = 16 elements: chunk, K step of 32, half of the step
    const int half = unit & 1, step = (unit >> 1) & 7, r = row & 127;
    const uint8_t* stg = a.w + ((size_t)(row >> 7) * a.row_bytes + (unit >> 4)) * kQ80Stage;
    uint4 q = ld_stream(reinterpret_cast<const uint4*>(stg + step * 4096 + half * 2048 + (r >> 3) * 128 + (r & 7) * 16));
    q.x ^= 0x80808080u;  // signed bytes here, q + 128 in the streaming layout the arithmetic expects
    q.y ^= 0x80808080u;
    q.z ^= 0x80808080u;
    q.w ^= 0x80808080u;
    t.q = q;
    t.d = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(stg + 128 * 256 + r * 16 + step * 2)));
  }
};

// ---- streaming layouts: the expert's rows once per four of its items ---------------------------
constexpr int kMaxWorkItems = 1024;  // items a CTA can collect for its expert
constexpr int kWorkM = 4;            // items per pass over the expert's rows

struct WorkArgs {
  const uint32_t* experts;  // [work_len] or nullptr (one expert)
  const uint32_t* pos;      // scatter: destination row of an item
  const float* weight;      // scatter: weight of an item
  int work_len, active_experts;
  int expert_rows;          // rows of one expert in the matrix (gate|up: 2 * inter)
  int inter;                // gate|up: rows of gate (and of up)
  float* out;               // gate|up: [work_len][inter]; scatter: dst
  unsigned long long dst_len;
  int* status;
};

// One pass over the expert's rows for the items s_items[base .. base + m_now), m_now <= M.
// MODE 0: out[w][i] = gelu(gate_i . x_w) * (up_i . x_w); MODE 1: dst[pos[w]][r] += weight[w] * (W_e[r] . x_w)
template <class F, int MODE, int M>
__device__ __forceinline__ void work_pass(const StreamArgs& a, const WorkArgs& wa, int e, const unsigned short* s_items, int base,
                                          int m_now, unsigned char* smem_raw) {
  constexpr int S = F::kSlots, R = 2;
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)M * a.iters * S * 32 * 16);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int iters = a.iters;
  // a task = two rows of the expert: gate row i and up row i, or two adjacent rows
  const int tasks = MODE == 0 ? wa.inter : (wa.expert_rows + 1) / 2;
  const int task_stride = gridDim.x * kGWarps;
  const int row0 = e * wa.expert_rows;
  int task = blockIdx.x * kGWarps + warp, it = 0;
  typename F::Row cur[R], nxt[R];
  auto load_tile = [&](int t, int i, typename F::Row (&dst)[R]) {
    int unit = i * 32 + lane;
    if (unit >= a.units) unit = a.units - 1;  // the staged x is zero there
    int row[R];
    if (MODE == 0) {
      row[0] = row0 + t;
      row[1] = row0 + wa.inter + t;
    } else {
      row[0] = row0 + 2 * t;
      row[1] = row0 + min(2 * t + 1, wa.expert_rows - 1);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) F::load(a, row[r], unit, dst[r]);
  };
  const bool has_work = task < tasks;
  if (has_work) load_tile(task, 0, cur);  // first weights in flight while the activations are staged
  {
    const int per_m = iters * S * 32, total = M * per_m;
    for (int idx = threadIdx.x; idx < total; idx += kGThreads) {
      const int m = idx / per_m, rem = idx - m * per_m;
      const int i = rem / (S * 32), slot = (rem >> 5) % S, l = rem & 31, unit = i * 32 + l;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < m_now && unit < a.units)
        v = __ldg(reinterpret_cast<const float4*>(a.x + (size_t)s_items[base + m] * a.in_dim + (size_t)unit * (S * 4) + slot * 4));
      xs[idx] = v;
    }
    __syncthreads();
    if (F::kHasConsts) {
      const int nsum = M * iters * 32;
      for (int idx = threadIdx.x; idx < nsum; idx += kGThreads) {
        const int mi = idx >> 5, l = idx & 31;
        float se = 0.f, so = 0.f;
#pragma unroll
        for (int sl = 0; sl < S; ++sl) {
          const float4 v = xs[(mi * S + sl) * 32 + l];
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
      for (int sl = 0; sl < S; ++sl) xv[m][sl] = xs[((size_t)(m * iters + it) * S + sl) * 32 + lane];
      c[m] = F::kHasConsts ? xc[(m * iters + it) * 32 + lane] : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) F::template dot<M>(cur[r], xv, c, acc[r]);
    if (it == iters - 1) {
      float v[R][M];
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          v[r][m] = warp_sum(acc[r][m]);
          acc[r][m] = 0.f;
        }
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          if (m >= m_now) continue;
          const int w = s_items[base + m];
          if (MODE == 0) {
            wa.out[(size_t)w * wa.inter + task] = gelu_tanh(v[0][m]) * v[1][m];
          } else {
            const float wt = wa.weight[w];
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const int lr = 2 * task + r;
              if (lr >= wa.expert_rows) continue;
              const unsigned long long at = (unsigned long long)wa.pos[w] * (unsigned long long)wa.expert_rows + (unsigned long long)lr;
              if (at < wa.dst_len) atomicAdd(wa.out + at, v[r][m] * wt);  // items may share a destination row
              else atomicCAS(wa.status, 0, 602);
            }
          }
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

// grid (row blocks, Y).  BY_ITEM (lists shorter than the number of experts): Y = items, and the CTAs
// of an item work for its expert if the item is the first of that expert in the list, else return;
// otherwise Y = experts.  Either way a CTA collects all items of its expert and passes over the
// expert's rows once per four of them.
template <class F, int MODE, bool BY_ITEM>
__global__ void __launch_bounds__(kGThreads)
stream_work_kernel(const __grid_constant__ StreamArgs a, const __grid_constant__ WorkArgs wa) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_n, s_dup;
  __shared__ unsigned short s_items[kMaxWorkItems];
  if (threadIdx.x == 0) s_n = s_dup = 0;
  __syncthreads();
  uint32_t e = blockIdx.y;
  if (BY_ITEM) {
    e = wa.experts ? wa.experts[blockIdx.y] : 0u;
    if (e >= (uint32_t)wa.active_experts) {
      if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(wa.status, 0, 601);
      return;
    }
    for (int w = threadIdx.x; w < (int)blockIdx.y; w += kGThreads)
      if ((wa.experts ? wa.experts[w] : 0u) == e) s_dup = 1;
    __syncthreads();
    if (s_dup) return;  // an earlier item's CTAs work for this expert
  }
  for (int w = threadIdx.x; w < wa.work_len; w += kGThreads) {
    const uint32_t we = wa.experts ? wa.experts[w] : 0u;
    if (we == e) s_items[atomicAdd(&s_n, 1)] = (unsigned short)w;
    else if (!BY_ITEM && we >= (uint32_t)wa.active_experts && e == 0 && blockIdx.x == 0) atomicCAS(wa.status, 0, 601);
  }
  __syncthreads();
  const int n = s_n;
  if (n == 1) {
    work_pass<F, MODE, 1>(a, wa, (int)e, s_items, 0, 1, smem_raw);
  } else if (n == 2) {
    work_pass<F, MODE, 2>(a, wa, (int)e, s_items, 0, 2, smem_raw);
  } else {
    for (int base = 0; base < n; base += kWorkM) {
      if (base) __syncthreads();  // every warp is done with the items before
      work_pass<F, MODE, kWorkM>(a, wa, (int)e, s_items, base, min(kWorkM, n - base), smem_raw);
    }
  }
}

// Launches the grouped form when the list fits a CTA's item table; false = not taken.
template <int MODE, class F>
static void (*pick_work_kernel(bool by_item))(const StreamArgs, const WorkArgs) {
  return by_item ? stream_work_kernel<F, MODE, true> : stream_work_kernel<F, MODE, false>;
}

template <int MODE>
bool launch_stream_work(const goph_gguf_matrix* m, const float* x, const WorkArgs& wa, cudaStream_t stream, int* rc) {
  if (wa.work_len > kMaxWorkItems || m->in_dim % 256) return false;
  StreamArgs a;
  memset(&a, 0, sizeof a);
  const bool q4 = m->qtype == GOPH_GGUF_Q4_K, tiled = m->tiled != nullptr;
  a.w = tiled ? m->tiled : m->data;
  a.aux = m->d16;
  a.x = x;
  a.rows = m->out_dim;
  a.in_dim = m->in_dim;
  a.units = q4 ? m->in_dim / 32 : m->in_dim / 16;
  a.iters = (a.units + 31) / 32;
  a.row_bytes = tiled ? m->in_dim / 256 : (q4 ? m->in_dim / 256 * 144 : m->in_dim);
  a.x_aligned = 1;
  const size_t smem = q4 ? stream_smem_bytes<Q4KFmt>(kWorkM, a.iters) : stream_smem_bytes<Q80Fmt>(kWorkM, a.iters);
  if (smem > (size_t)kSmemBudget) return false;
  const bool by_item = wa.work_len < wa.active_experts;
  auto kern = q4 ? (tiled ? pick_work_kernel<MODE, Q4KTiledFmt>(by_item) : pick_work_kernel<MODE, Q4KFmt>(by_item))
                 : (tiled ? pick_work_kernel<MODE, Q80TiledFmt>(by_item) : pick_work_kernel<MODE, Q80Fmt>(by_item));
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    *rc = fail_cuda(cudaGetLastError(), "cudaFuncSetAttribute(work-list kernel)");
    return true;
  }
  const int tasks = MODE == 0 ? wa.inter : (wa.expert_rows + 1) / 2;
  const int live = wa.active_experts < wa.work_len ? wa.active_experts : wa.work_len;  // experts that can have items
  const int sms = device_state(m->device).sm_count;
  int gx = (4 * sms + live - 1) / live;
  const int max_gx = (tasks + kGWarps - 1) / kGWarps;
  if (gx > max_gx) gx = max_gx;
  if (gx < 1) gx = 1;
  note_launch();
  kern<<<dim3(gx, by_item ? wa.work_len : wa.active_experts), kGThreads, smem, stream>>>(a, wa);
  cudaError_t e = cudaGetLastError();
  *rc = e == cudaSuccess ? GOPH_OK : fail_cuda(e, "work-list kernel launch");
  return true;
}

int* work_status(int device) {
  static int* words[kMaxDevices] = {};
  static std::mutex mu;
  if (device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!words[device]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess || cudaMemset(p, 0, sizeof(int)) != cudaSuccess) {
      cudaFree(p);
      cudaGetLastError();
      return nullptr;
    }
    words[device] = p;
  }
  return words[device];
}

bool valid_work_matrix(const goph_gguf_matrix* m) {
  return m && m->magic == kMagicGGUF && (m->qtype == GOPH_GGUF_Q4_K || m->qtype == GOPH_GGUF_Q8_0) && m->in_dim > 0 &&
         m->in_dim % 32 == 0 && m->out_dim > 0 && (m->tiled || m->data);
}

WorkView view_of(const goph_gguf_matrix* m) {
  WorkView v;
  v.data = m->data;
  v.d16 = m->d16;
  v.tiled = m->tiled;
  v.qtype = m->qtype;
  v.in_dim = m->in_dim;
  v.out_dim = m->out_dim;
  v.nchunks = m->in_dim / 256;
  return v;
}

}  // namespace

int gguf_work_status(int device) {
  int* p = work_status(device);
  if (!p) return 0;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return v;
}

void gguf_work_status_clear(int device) {
  int* p = work_status(device);
  if (p) cudaMemset(p, 0, sizeof(int));
}

}  // namespace goph

using namespace goph;

GOPH_API int goph_gguf_gate_up_gelu_by_work(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len,
                                            const uint32_t* work_experts_dev, int work_len, int intermediate, int active_experts,
                                            const goph_gguf_matrix* m, void* stream) {
  clear_error();
  if (work_len <= 0) return GOPH_OK;  // as the reference: nothing to do
  if (!valid_work_matrix(m)) return fail(GOPH_E_INVALID, "gate/up by work: a Q4_K or Q8_0 matrix handle is required");
  uint64_t need_x, need_o, need_rows;
  if (intermediate <= 0 || active_experts <= 0 || !mul_ok((uint64_t)work_len, (uint64_t)m->in_dim, &need_x) ||
      !mul_ok((uint64_t)work_len, (uint64_t)intermediate, &need_o) ||
      !mul_ok((uint64_t)active_experts, 2ull * (uint64_t)intermediate, &need_rows) || (uint64_t)m->out_dim < need_rows)
    return fail(GOPH_E_INVALID, "gate/up by work: intermediate=%d experts=%d against %d rows", intermediate, active_experts, m->out_dim);
  if (!x_dev || x_len < need_x || !out_dev || out_len < need_o || (active_experts > 1 && !work_experts_dev))
    return fail(GOPH_E_INVALID, "gate/up by work buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len,
                (unsigned long long)need_x, (unsigned long long)out_len, (unsigned long long)need_o);
  if ((uintptr_t)x_dev % 16) return fail(GOPH_E_INVALID, "x must be 16-byte aligned");
  if (int rc = use_device(m->device)) return rc;
  int* status = work_status(m->device);
  if (!status) return fail(GOPH_E_NOMEM, "cannot allocate the work-list kernels' status word");
  {
    WorkArgs wa;
    memset(&wa, 0, sizeof wa);
    wa.experts = work_experts_dev;
    wa.work_len = work_len;
    wa.active_experts = active_experts;
    wa.expert_rows = 2 * intermediate;
    wa.inter = intermediate;
    wa.out = out_dev;
    wa.status = status;
    int rc = GOPH_OK;
    if (launch_stream_work<0>(m, x_dev, wa, (cudaStream_t)stream, &rc)) return rc;
  }
  note_launch();
  gate_up_gelu_kernel<<<dim3((intermediate + kWarps - 1) / kWarps, work_len), kWarps * 32, 0, (cudaStream_t)stream>>>(
      view_of(m), x_dev, work_experts_dev, active_experts, intermediate, out_dev, status);
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

GOPH_API int goph_gguf_gate_up_gelu(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len, int batch,
                                    int intermediate, const goph_gguf_matrix* m, void* stream) {
  if (m && m->magic == kMagicGGUF && intermediate > 0 && m->out_dim != 2 * intermediate) {
    clear_error();
    return fail(GOPH_E_INVALID, "gate/up: the matrix has %d rows, not 2 x %d", m->out_dim, intermediate);
  }
  return goph_gguf_gate_up_gelu_by_work(out_dev, out_len, x_dev, x_len, nullptr, batch, intermediate, 1, m, stream);
}

GOPH_API int goph_gguf_scatter_by_work(float* dst_dev, uint64_t dst_len, const float* x_dev, uint64_t x_len,
                                       const uint32_t* work_active_dev, const uint32_t* work_pos_dev,
                                       const float* work_weight_dev, int work_len, int active_experts,
                                       const goph_gguf_matrix* m, void* stream) {
  clear_error();
  if (work_len <= 0) return GOPH_OK;
  if (!valid_work_matrix(m)) return fail(GOPH_E_INVALID, "scatter by work: a Q4_K or Q8_0 matrix handle is required");
  uint64_t need_x;
  if (active_experts <= 0 || m->out_dim % active_experts != 0 || !mul_ok((uint64_t)work_len, (uint64_t)m->in_dim, &need_x))
    return fail(GOPH_E_INVALID, "scatter by work: %d rows do not divide into %d experts", m->out_dim, active_experts);
  if (!x_dev || x_len < need_x || !dst_dev || dst_len == 0 || !work_pos_dev || !work_weight_dev ||
      (active_experts > 1 && !work_active_dev))
    return fail(GOPH_E_INVALID, "scatter by work buffers x=%llu/%llu", (unsigned long long)x_len, (unsigned long long)need_x);
  if ((uintptr_t)x_dev % 16) return fail(GOPH_E_INVALID, "x must be 16-byte aligned");
  if (int rc = use_device(m->device)) return rc;
  int* status = work_status(m->device);
  if (!status) return fail(GOPH_E_NOMEM, "cannot allocate the work-list kernels' status word");
  const int expert_out = m->out_dim / active_experts;
  {
    WorkArgs wa;
    memset(&wa, 0, sizeof wa);
    wa.experts = work_active_dev;
    wa.pos = work_pos_dev;
    wa.weight = work_weight_dev;
    wa.work_len = work_len;
    wa.active_experts = active_experts;
    wa.expert_rows = expert_out;
    wa.out = dst_dev;
    wa.dst_len = (unsigned long long)dst_len;
    wa.status = status;
    int rc = GOPH_OK;
    if (launch_stream_work<1>(m, x_dev, wa, (cudaStream_t)stream, &rc)) return rc;
  }
  note_launch();
  scatter_by_work_kernel<<<dim3((expert_out + kWarps - 1) / kWarps, work_len), kWarps * 32, 0, (cudaStream_t)stream>>>(
      view_of(m), x_dev, work_active_dev, work_pos_dev, work_weight_dev, active_experts, expert_out, dst_dev,
      (unsigned long long)dst_len, status);
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

GOPH_API int goph_gguf_project_scatter(float* dst_dev, uint64_t dst_len, const float* x_dev, uint64_t x_len,
                                       const uint32_t* pos_dev, const float* weight_dev, int batch, const goph_gguf_matrix* m,
                                       void* stream) {
  return goph_gguf_scatter_by_work(dst_dev, dst_len, x_dev, x_len, nullptr, pos_dev, weight_dev, batch, 1, m, stream);
}
