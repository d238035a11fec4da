// The operations of a decode step that are not matrix products: RMSNorm (with the residual add in
// front of it), per-head QK RMSNorm + RoPE + KV append, grouped-query attention over the KV cache,
// SiLU*up, argmax, embedding lookup from the tied 4-bit LM head, position bookkeeping.
//
// Replaces the decode-step kernels of GPUModel.Generate (model/gpu_forward.go:993-1357: rms_norm,
// rope, attention_score / softmax / attention_out, silu_mul, add, argmax); arithmetic specification:
// runLegacyCPUToken (model/llama.go:899-1441) with simd.RMSNorm, kernels.ApplyRoPE,
// simd.GQAAttentionScaleInto, kernels.SiLU and ArgmaxLogits (model/inference_helpers.go:248-261).
// The position and the current token live in device memory (`pos_dev`, `tok_dev`) and the kernels
// read them there, so one captured CUDA graph serves every step of a generation.
// Every kernel starts with the programmatic-dependent-launch prologue used across the library.
#include <math_constants.h>
#include <string.h>

#include <mutex>

#include "goph_internal.cuh"
#include "mlx_mma.cuh"

namespace goph {

__device__ __forceinline__ void pdl_begin() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += sh[i];
  return t;
}

// hidden = a (+ b); normed = (hidden * inv) * w, inv = 1/sqrt(sum(hidden^2)/n + eps).  One CTA per
// row; rows of up to 2048 elements stay in registers between the two passes.
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(float* hidden, float* __restrict__ normed, const float* a, const float* __restrict__ b,
                   const float* __restrict__ w, int n, float eps) {
  __shared__ float sh[8];
  pdl_begin();
  const size_t row = blockIdx.x;
  constexpr int kKeep = 8;
  const bool keep = n <= 256 * kKeep;
  float v[kKeep];
  float ss = 0.f;
  if (keep) {
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
      const int i = threadIdx.x + j * 256;
      v[j] = 0.f;
      if (i < n) {
        v[j] = a[row * n + i];
        if (b) v[j] = __fadd_rn(v[j], b[row * n + i]);
      }
    }
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < n && hidden) hidden[row * n + i] = v[j];
      ss = fmaf(v[j], v[j], ss);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float x = a[row * n + i];
      if (b) x = __fadd_rn(x, b[row * n + i]);
      if (hidden) hidden[row * n + i] = x;
      ss = fmaf(x, x, ss);
    }
  }
  ss = block_sum(ss, sh);
  const float inv = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)n), eps)));
  if (keep) {
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < n) normed[row * n + i] = __fmul_rn(__fmul_rn(v[j], inv), w[i]);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float x;
      if (hidden) {
        x = hidden[row * n + i];  // written above by this thread (hidden may be the same buffer as a)
      } else {
        x = a[row * n + i];
        if (b) x = __fadd_rn(x, b[row * n + i]);
      }
      normed[row * n + i] = __fmul_rn(__fmul_rn(x, inv), w[i]);
    }
  }
}

// Set when a kernel found the position word outside [0, max_seq): 401 the KV append, 402 attention.
// Such a kernel touches neither the caches nor its output (a step replayed once more than the cache
// holds, or a stale position word, must not write out of bounds).  Read through goph_kernel_status.
__device__ int g_decode_status;

// Per head (q heads then k heads): optional RMSNorm with the head-dim weight, RoPE on the pairs
// (i, i + d/2) with the table row of *pos_dev; q in place, k into the cache row, v copied into its
// cache row.  One CTA of head_dim/2 threads per head; head_dim <= 512.
__global__ void __launch_bounds__(256)
qk_norm_rope_append_kernel(float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                           const float* __restrict__ qw, const float* __restrict__ kw,
                           const float* __restrict__ table, const int* __restrict__ pos_dev,
                           float* __restrict__ kcache, float* __restrict__ vcache, int heads, int kv_heads,
                           int head_dim, float eps, int max_seq) {
  __shared__ float sh[8];
  pdl_begin();
  const int pos = *pos_dev, half = head_dim / 2, i = threadIdx.x;
  if (pos < 0 || pos >= max_seq) {
    if (i == 0) atomicCAS(&g_decode_status, 0, 401);
    return;
  }
  const bool is_q = (int)blockIdx.x < heads;
  const int head = is_q ? blockIdx.x : blockIdx.x - heads;
  const float* src = (is_q ? q : k) + (size_t)head * head_dim;
  float x0 = src[i], x1 = src[i + half];
  const float* w = is_q ? qw : kw;
  if (w) {
    float ss = block_sum(fmaf(x0, x0, x1 * x1), sh);
    const float inv = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)head_dim), eps)));
    x0 = __fmul_rn(__fmul_rn(x0, inv), w[i]);
    x1 = __fmul_rn(__fmul_rn(x1, inv), w[i + half]);
  }
  const float c = table[((size_t)pos * half + i) * 2], s = table[((size_t)pos * half + i) * 2 + 1];
  const float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
  const float y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
  const size_t kvd = (size_t)kv_heads * head_dim;
  if (is_q) {
    q[(size_t)head * head_dim + i] = y0;
    q[(size_t)head * head_dim + i + half] = y1;
  } else {
    float* kd = kcache + (size_t)pos * kvd + (size_t)head * head_dim;
    kd[i] = y0;
    kd[i + half] = y1;
    float* vd = vcache + (size_t)pos * kvd + (size_t)head * head_dim;
    const float* vs = v + (size_t)head * head_dim;
    vd[i] = vs[i];
    vd[i + half] = vs[i + half];
  }
}

// Grid (query heads, position splits): a CTA of W warps takes every split-th block of
// W*4 positions of its head.  Scores: a warp takes four positions at a time so their K and V
// rows are all in flight together (the V rows are requested before the softmax); the CTA's softmax
// numerators use its own maximum; a warp accumulates e_t * v_t for all of head_dim (lane d, d+32, ..).
// One split (sequences up to a few hundred positions): the CTA writes the head's output.  Several
// splits: each leaves {max, sum, vector} in global scratch and the head's last CTA merges them,
// out = sum_s a_s v_s / sum_s a_s l_s with a_s = exp(m_s - m).
// FUSED: the kernel also does what qk_norm_rope_append_kernel does — every warp norms and rotates
// its head's q for itself; the warp that owns the current position norms and rotates the new k,
// uses it and the new v from the projection output instead of the cache, and (for the first head
// of a KV group) writes both into the cache rows.  No CTA reads the cache row being written.
constexpr int kAttnMaxSplits = 16, kAttnMaxHeads = 256;

template <int EPL>
__device__ __forceinline__ void norm_rope_head(float (&x)[EPL], const float* __restrict__ w, const float* __restrict__ trow,
                                               int head_dim, float eps, int lane) {
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) ss = fmaf(x[e], x[e], ss);
    ss = warp_sum(ss);
    const float inv = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)head_dim), eps)));
#pragma unroll
    for (int e = 0; e < EPL; ++e) x[e] = __fmul_rn(__fmul_rn(x[e], inv), w[lane + 32 * e]);
  }
#pragma unroll
  for (int e = 0; e < EPL / 2; ++e) {  // pairs (i, i + head_dim/2) sit in the same lane
    const int i = lane + 32 * e;
    const float c = trow[2 * i], sn = trow[2 * i + 1];
    const float x0 = x[e], x1 = x[e + EPL / 2];
    x[e] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
    x[e + EPL / 2] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
  }
}

struct AttnArgs {
  float* out;
  const float* q;        // FUSED: raw projection output; else already normed and rotated
  const float* k_new;    // FUSED: raw k and v of the current position
  const float* v_new;
  const float* q_norm;   // FUSED: head-dim RMSNorm weights or null
  const float* k_norm;
  const float* table;    // FUSED: RoPE table [max_seq][head_dim/2][2]
  float* kcache;
  float* vcache;
  const int* pos_dev;
  int heads, kv_heads, head_dim;
  int max_seq;           // rows of the caches and of the RoPE table
  float scale, eps;
  float* scratch;
  unsigned int* counters;
};

template <int EPL, bool FUSED, int W>
__global__ void __launch_bounds__(W * 32)
attn_decode_kernel(const __grid_constant__ AttnArgs a) {
  extern __shared__ float scores[];
  __shared__ float sh[W];
  __shared__ float part[W][EPL * 32];
  __shared__ int s_last;
  pdl_begin();
  const int pos = *a.pos_dev, seq = pos + 1;
  if (pos < 0 || pos >= a.max_seq) {
    if (threadIdx.x == 0) atomicCAS(&g_decode_status, 0, 402);
    return;
  }
  const int heads = a.heads, kv_heads = a.kv_heads, head_dim = a.head_dim;
  const int head = blockIdx.x, per = heads / kv_heads, kvh = head / per;
  const int splits = gridDim.y, split = blockIdx.y;
  const size_t kvd = (size_t)kv_heads * head_dim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* kbase = a.kcache + (size_t)kvh * head_dim;
  const float* vbase = a.vcache + (size_t)kvh * head_dim;
  constexpr int B = 4 * W;
  const int nblocks = (seq + B - 1) / B;
  const int my_blocks = nblocks > split ? (nblocks - split + splits - 1) / splits : 0;
  auto pos_of = [&](int i) { return ((i / B) * splits + split) * B + (i % B); };
  const int nloc = my_blocks * B;  // local indices (some past seq in the last block)
  float qr[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) qr[e] = a.q[(size_t)head * head_dim + lane + 32 * e];
  if (FUSED) norm_rope_head<EPL>(qr, a.q_norm, a.table + (size_t)pos * head_dim, head_dim, a.eps, lane);
  float acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
  // One block of positions per iteration; with several iterations the accumulators are rescaled to
  // the running maximum (the usual single-pass softmax); the common case is one iteration.
  float run_max = -CUDART_INF_F, run_sum = 0.f;
  for (int blk = 0; blk < my_blocks; ++blk) {
    float kv_k[4][EPL], kv_v[4][EPL];
    int tt[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = pos_of(blk * B + warp + j * W);
      tt[j] = t;
      const bool cur = FUSED && t == pos;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const size_t off = (size_t)t * kvd + lane + 32 * e;
        kv_k[j][e] = t < seq ? (cur ? a.k_new[(size_t)kvh * head_dim + lane + 32 * e] : kbase[off]) : 0.f;
        kv_v[j][e] = t < seq ? (cur ? a.v_new[(size_t)kvh * head_dim + lane + 32 * e] : vbase[off]) : 0.f;
      }
    }
    float sc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (FUSED && tt[j] == pos) {  // the new position: norm, rotate, and (one warp per KV head) append
        norm_rope_head<EPL>(kv_k[j], a.k_norm, a.table + (size_t)pos * head_dim, head_dim, a.eps, lane);
        if (head % per == 0) {
#pragma unroll
          for (int e = 0; e < EPL; ++e) {
            a.kcache[(size_t)pos * kvd + (size_t)kvh * head_dim + lane + 32 * e] = kv_k[j][e];
            a.vcache[(size_t)pos * kvd + (size_t)kvh * head_dim + lane + 32 * e] = kv_v[j][e];
          }
        }
      }
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) d = fmaf(qr[e], kv_k[j][e], d);
      d = warp_sum(d);
      sc[j] = tt[j] < seq ? __fmul_rn(d, a.scale) : -CUDART_INF_F;
    }
    // block maximum
    float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
    if (lane == 0) sh[warp] = mx;
    __syncthreads();
    mx = sh[0];
#pragma unroll
    for (int i = 1; i < W; ++i) mx = fmaxf(mx, sh[i]);
    const float new_max = fmaxf(run_max, mx);
    // single-precision exp (2 ulp) where the reference rounds an f64 exp to f32: the FP64 pipe of
    // this part is too slow for a per-position operation
    const float rescale = run_max == -CUDART_INF_F ? 0.f : expf(run_max - new_max);
    float local = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] *= rescale;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p = sc[j] == -CUDART_INF_F ? 0.f : expf(sc[j] - new_max);
      local += p;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[e] = fmaf(p, kv_v[j][e], acc[e]);
    }
    __syncthreads();  // sh is reused
    if (lane == 0) sh[warp] = local;   // every lane of the warp holds the same four p: one copy per warp
    __syncthreads();
    float bsum = 0.f;
#pragma unroll
    for (int i = 0; i < W; ++i) bsum += sh[i];
    run_sum = fmaf(run_sum, rescale, bsum);
    run_max = new_max;
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) part[warp][lane + 32 * e] = acc[e];
  __syncthreads();
  if (splits == 1) {
    const float inv = __fdiv_rn(1.f, run_sum);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
      float r = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) r += part[w][d];
      a.out[(size_t)head * head_dim + d] = __fmul_rn(r, inv);
    }
    return;
  }
  // ---- this split's {max, sum, vector} to scratch; the head's last CTA merges -------------------
  const int stride = 2 + 256;
  float* mine = a.scratch + ((size_t)head * kAttnMaxSplits + split) * stride;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float r = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) r += part[w][d];
    mine[2 + d] = r;
  }
  if (threadIdx.x == 0) {
    mine[0] = run_max;
    mine[1] = run_sum;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(a.counters + head, 1u) == (unsigned)splits - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* base = a.scratch + (size_t)head * kAttnMaxSplits * stride;
  // the splits' rescaling factors a_s = exp(m_s - m), computed once
  __shared__ float fac[kAttnMaxSplits];
  __shared__ float s_inv;
  if (threadIdx.x < 32) {
    float m = -CUDART_INF_F;
    for (int s2 = 0; s2 < splits; ++s2) m = fmaxf(m, __ldcg(base + s2 * stride));
    float mine_f = 0.f;
    if (lane < splits) {
      const float ms = __ldcg(base + lane * stride);
      mine_f = ms == -CUDART_INF_F ? 0.f : expf(ms - m);
      fac[lane] = mine_f;
    }
    float total = lane < splits ? __fmul_rn(__ldcg(base + lane * stride + 1), mine_f) : 0.f;
    total = warp_sum(total);
    if (lane == 0) s_inv = __fdiv_rn(1.f, total);
  }
  __syncthreads();
  const float inv = s_inv;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float r = 0.f;
    for (int s2 = 0; s2 < splits; ++s2) r = fmaf(__ldcg(base + s2 * stride + 2 + d), fac[s2], r);
    a.out[(size_t)head * head_dim + d] = __fmul_rn(r, inv);
  }
  if (threadIdx.x == 0) a.counters[head] = 0;
}

// out[i] = silu(gate[i]) * up[i]; gate and up are the two halves of one fused projection output.
__global__ void silu_mul_kernel(float* __restrict__ out, const float* __restrict__ gate, const float* __restrict__ up, int n) {
  pdl_begin();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float g = gate[i];
  out[i] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.f, expf(-g))), up[i]);  // expf: see attn_decode_kernel
}

// First maximum of logits[0..n): kArgmaxCtas CTAs reduce a slice each; the last one to arrive
// reduces their results, and the winner becomes the current token and the position advances by one
// (the bookkeeping of the greedy loop, model/llama.go:826-895).  scratch: kArgmaxCtas {value, index}
// pairs and an arrival counter that the last CTA leaves at zero.
constexpr int kArgmaxCtas = 64;
__device__ __forceinline__ void argmax_merge(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) {
    best = ov;
    bi = oi;
  }
}
__global__ void __launch_bounds__(512)
argmax_advance_kernel(const float* __restrict__ logits, int n, int* __restrict__ tok_dev, int* __restrict__ pos_dev,
                      int* __restrict__ history, const int* __restrict__ forced, int history_cap,
                      float* __restrict__ part_val, int* __restrict__ part_idx, unsigned int* __restrict__ counter) {
  __shared__ float sv[16];
  __shared__ int si[16];
  __shared__ int s_last;
  pdl_begin();
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int lo = blockIdx.x * per, hi = min(n, lo + per);
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = logits[i];
    if (v > best) {  // ascending scan: within a thread the first maximum wins
      best = v;
      bi = i;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o; o >>= 1) argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < nw; ++w) argmax_merge(best, bi, sv[w], si[w]);
    part_val[blockIdx.x] = best;
    part_idx[blockIdx.x] = bi;
    __threadfence();
    s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last || threadIdx.x >= 32) return;
  __threadfence();
  best = -CUDART_INF_F;
  bi = 0x7fffffff;
  for (int c = lane; c < (int)gridDim.x; c += 32) argmax_merge(best, bi, __ldcg(part_val + c), __ldcg(part_idx + c));
#pragma unroll
  for (int o = 16; o; o >>= 1) argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane == 0) {
    if (bi == 0x7fffffff) bi = 0;  // all NaN: ArgmaxLogits keeps index 0
    const int pos = *pos_dev;
    // while the prompt is being fed the next token is given, not chosen
    if (forced && pos + 1 < history_cap && forced[pos + 1] >= 0) bi = forced[pos + 1];
    *tok_dev = bi;
    if (history && pos + 1 < history_cap) history[pos + 1] = bi;
    *pos_dev = pos + 1;
    *counter = 0;
  }
}

// hidden = dequantised row *tok_dev of an MLX weight (the tied LM head used as embedding table,
// LlamaModel.TokenEmbeddingInto), either layout.
__global__ void embed_mlx_kernel(float* __restrict__ out, const uint32_t* __restrict__ qweight, const void* __restrict__ sb,
                                 const unsigned char* __restrict__ tiled, const int* __restrict__ tok_dev, int in_dim,
                                 int group_size, int sb_bf16) {
  pdl_begin();
  const int row = *tok_dev;
  const int word = blockIdx.x * blockDim.x + threadIdx.x;  // packed word index within the row
  if (word >= in_dim / 8) return;
  const int col = word * 8, groups = in_dim / group_size, g = col / group_size;
  uint32_t w;
  float sc, bi;
  if (tiled) {
    const int nchunks = in_dim / kMlxChunkK;
    w = *reinterpret_cast<const uint32_t*>(tiled + mlx_tiled_word_offset(row, col, nchunks));
    const uint32_t m = *reinterpret_cast<const uint32_t*>(tiled + mlx_tiled_meta_offset(row, col, nchunks));
    sc = __uint_as_float(m << 16);
    bi = __uint_as_float(m & 0xFFFF0000u);
  } else {
    w = qweight[(size_t)row * (in_dim / 8) + word];
    if (sb_bf16) {
      const uint32_t m = reinterpret_cast<const uint32_t*>(sb)[(size_t)row * groups + g];
      sc = __uint_as_float(m << 16);
      bi = __uint_as_float(m & 0xFFFF0000u);
    } else {
      const float2 m = reinterpret_cast<const float2*>(sb)[(size_t)row * groups + g];
      sc = m.x;
      bi = m.y;
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) out[col + e] = __fadd_rn(__fmul_rn((float)((w >> (4 * e)) & 0xF), sc), bi);
}

template <typename... KArgs, typename... Args>
static int op_launch(void (*k)(KArgs...), dim3 grid, int threads, size_t smem, void* stream, Args... args) {
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  note_launch();
  GOPH_CUDA(cudaLaunchKernelEx(&cfg, k, KArgs(args)...));
  return GOPH_OK;
}

}  // namespace goph

namespace goph {
int decode_ops_status() {
  int v = 0;
  return cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) == cudaSuccess ? v : -1;
}
void decode_ops_status_clear() {
  const int zero = 0;
  cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
}
}  // namespace goph

using namespace goph;

GOPH_API int goph_add_rmsnorm(int device, float* hidden_dev, float* normed_dev, const float* a_dev, const float* b_dev,
                              const float* weight_dev, int n, int rows, float eps, void* stream) {
  clear_error();
  if (!normed_dev || !a_dev || !weight_dev || n <= 0 || rows <= 0) return fail(GOPH_E_INVALID, "goph_add_rmsnorm: n=%d rows=%d", n, rows);
  if (int rc = use_device(device)) return rc;
  return op_launch(add_rmsnorm_kernel, dim3(rows), 256, 0, stream, hidden_dev, normed_dev, a_dev, b_dev, weight_dev, n, eps);
}

GOPH_API int goph_qk_norm_rope_append(int device, float* q_dev, const float* k_dev, const float* v_dev,
                                      const float* q_norm_dev, const float* k_norm_dev, const float* rope_table_dev,
                                      const int* pos_dev, float* kcache_dev, float* vcache_dev, int max_seq, int heads,
                                      int kv_heads, int head_dim, float eps, void* stream) {
  clear_error();
  if (max_seq <= 0) return fail(GOPH_E_INVALID, "max_seq=%d", max_seq);
  if (!q_dev || !k_dev || !v_dev || !rope_table_dev || !pos_dev || !kcache_dev || !vcache_dev)
    return fail(GOPH_E_INVALID, "goph_qk_norm_rope_append: nil buffer");
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || head_dim < 64 || head_dim > 512 || head_dim % 64)
    return fail(GOPH_E_UNSUPPORTED, "attention dims heads=%d kv_heads=%d head_dim=%d (head_dim a multiple of 64 up to 512)", heads,
                kv_heads, head_dim);
  if ((q_norm_dev == nullptr) != (k_norm_dev == nullptr)) return fail(GOPH_E_INVALID, "QNorm without KNorm");
  if (int rc = use_device(device)) return rc;
  return op_launch(qk_norm_rope_append_kernel, dim3(heads + kv_heads), head_dim / 2, 0, stream, q_dev, k_dev, v_dev, q_norm_dev,
                   k_norm_dev, rope_table_dev, pos_dev, kcache_dev, vcache_dev, heads, kv_heads, head_dim, eps, max_seq);
}

static int attn_launch(int device, AttnArgs& a, int max_seq, bool fused, void* stream) {
  if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads || a.head_dim < 64 || a.head_dim > 256 || a.head_dim % 64)
    return fail(GOPH_E_UNSUPPORTED, "attention dims heads=%d kv_heads=%d head_dim=%d (head_dim 64, 128 or 256)", a.heads,
                a.kv_heads, a.head_dim);
  if (a.head_dim == 192) return fail(GOPH_E_UNSUPPORTED, "head_dim 192");
  if (a.heads > kAttnMaxHeads) return fail(GOPH_E_UNSUPPORTED, "at most %d query heads", kAttnMaxHeads);
  if (max_seq <= 0) return fail(GOPH_E_INVALID, "max_seq=%d", max_seq);
  if (int rc = use_device(device)) return rc;
  // Per-device scratch, allocated once.  Calls may come from any thread: the first calls are
  // serialised, and the pointers are published only when every allocation and the clearing of the
  // counters have succeeded (a failed first call leaves nothing half-made for the next one).
  static std::mutex mu;
  static float* scratch[kMaxDevices] = {};
  static unsigned int* counters[kMaxDevices] = {};
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!counters[device]) {
      float* s = nullptr;
      unsigned int* c = nullptr;
      if (cudaMalloc(&s, (size_t)kAttnMaxHeads * kAttnMaxSplits * (2 + 256) * sizeof(float)) != cudaSuccess ||
          cudaMalloc(&c, kAttnMaxHeads * sizeof(unsigned int)) != cudaSuccess ||
          cudaMemset(c, 0, kAttnMaxHeads * sizeof(unsigned int)) != cudaSuccess) {
        cudaFree(s);
        cudaFree(c);
        cudaGetLastError();
        return fail(GOPH_E_NOMEM, "cannot allocate the attention kernel's device scratch");
      }
      scratch[device] = s;
      counters[device] = c;
    }
    a.scratch = scratch[device];
    a.counters = counters[device];
  }
  a.max_seq = max_seq;
  // Short caches (the latency-bound case): CTAs of 4 warps, one block of 16 positions each, so that they
  // fit beside the projection kernels' CTAs and start under programmatic dependent launch (measured on
  // the Qwen3-0.6B step at positions 128-191: 1318 tok/s against 1249 with 32-warp CTAs).  Long caches:
  // CTAs of 32 warps, two blocks of 128 positions each without help, more through splits.
  const bool small = max_seq <= 16 * kAttnMaxSplits;
  const int per_cta = small ? 16 : 256;
  int splits = (max_seq + per_cta - 1) / per_cta;
  if (splits > kAttnMaxSplits) splits = kAttnMaxSplits;
  if (splits < 1) splits = 1;
  const dim3 grid(a.heads, splits);
#define GOPH_ATTN(EPL)                                                                                          \
  return small ? (fused ? op_launch(attn_decode_kernel<EPL, true, 4>, grid, 4 * 32, 0, stream, a)               \
                        : op_launch(attn_decode_kernel<EPL, false, 4>, grid, 4 * 32, 0, stream, a))             \
               : (fused ? op_launch(attn_decode_kernel<EPL, true, 32>, grid, 32 * 32, 0, stream, a)             \
                        : op_launch(attn_decode_kernel<EPL, false, 32>, grid, 32 * 32, 0, stream, a))
  if (a.head_dim == 64) GOPH_ATTN(2);
  if (a.head_dim == 128) GOPH_ATTN(4);
  GOPH_ATTN(8);
#undef GOPH_ATTN
}

GOPH_API int goph_attn_decode(int device, float* out_dev, const float* q_dev, const float* kcache_dev,
                              const float* vcache_dev, const int* pos_dev, int max_seq, int heads, int kv_heads,
                              int head_dim, float scale, void* stream) {
  clear_error();
  if (!out_dev || !q_dev || !kcache_dev || !vcache_dev || !pos_dev) return fail(GOPH_E_INVALID, "goph_attn_decode: nil buffer");
  AttnArgs a;
  memset(&a, 0, sizeof a);
  a.out = out_dev;
  a.q = q_dev;
  a.kcache = const_cast<float*>(kcache_dev);
  a.vcache = const_cast<float*>(vcache_dev);
  a.pos_dev = pos_dev;
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.scale = scale;
  return attn_launch(device, a, max_seq, false, stream);
}

GOPH_API int goph_attn_decode_fused(int device, float* out_dev, const float* q_dev, const float* k_dev, const float* v_dev,
                                    const float* q_norm_dev, const float* k_norm_dev, const float* rope_table_dev,
                                    const int* pos_dev, float* kcache_dev, float* vcache_dev, int max_seq, int heads,
                                    int kv_heads, int head_dim, float scale, float eps, void* stream) {
  clear_error();
  if (!out_dev || !q_dev || !k_dev || !v_dev || !rope_table_dev || !kcache_dev || !vcache_dev || !pos_dev)
    return fail(GOPH_E_INVALID, "goph_attn_decode_fused: nil buffer");
  if ((q_norm_dev == nullptr) != (k_norm_dev == nullptr)) return fail(GOPH_E_INVALID, "QNorm without KNorm");
  AttnArgs a;
  memset(&a, 0, sizeof a);
  a.out = out_dev;
  a.q = q_dev;
  a.k_new = k_dev;
  a.v_new = v_dev;
  a.q_norm = q_norm_dev;
  a.k_norm = k_norm_dev;
  a.table = rope_table_dev;
  a.kcache = kcache_dev;
  a.vcache = vcache_dev;
  a.pos_dev = pos_dev;
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.scale = scale;
  a.eps = eps;
  return attn_launch(device, a, max_seq, true, stream);
}

GOPH_API int goph_silu_mul(int device, float* out_dev, const float* gate_dev, const float* up_dev, int n, void* stream) {
  clear_error();
  if (!out_dev || !gate_dev || !up_dev || n <= 0) return fail(GOPH_E_INVALID, "goph_silu_mul: n=%d", n);
  if (int rc = use_device(device)) return rc;
  return op_launch(silu_mul_kernel, dim3((n + 255) / 256), 256, 0, stream, out_dev, gate_dev, up_dev, n);
}

GOPH_API int goph_argmax_advance(int device, const float* logits_dev, int n, int* tok_dev, int* pos_dev, int* history_dev,
                                 const int* forced_dev, int history_cap, void* stream) {
  clear_error();
  if (!logits_dev || n <= 0 || !tok_dev || !pos_dev) return fail(GOPH_E_INVALID, "goph_argmax_advance: n=%d", n);
  if (int rc = use_device(device)) return rc;
  // per-device scratch of the two-level reduction, allocated once
  static std::mutex mu;
  static float* part_val[kMaxDevices] = {};
  static int* part_idx[kMaxDevices] = {};
  static unsigned int* counter[kMaxDevices] = {};
  float* pv;
  int* pi;
  unsigned int* cnt;
  {
    std::lock_guard<std::mutex> lock(mu);  // as for the attention scratch: complete or not at all
    if (!counter[device]) {
      float* v = nullptr;
      int* i = nullptr;
      unsigned int* c = nullptr;
      if (cudaMalloc(&v, kArgmaxCtas * sizeof(float)) != cudaSuccess || cudaMalloc(&i, kArgmaxCtas * sizeof(int)) != cudaSuccess ||
          cudaMalloc(&c, sizeof(unsigned int)) != cudaSuccess || cudaMemset(c, 0, sizeof(unsigned int)) != cudaSuccess) {
        cudaFree(v);
        cudaFree(i);
        cudaFree(c);
        cudaGetLastError();
        return fail(GOPH_E_NOMEM, "cannot allocate the argmax kernel's device scratch");
      }
      part_val[device] = v;
      part_idx[device] = i;
      counter[device] = c;
    }
    pv = part_val[device];
    pi = part_idx[device];
    cnt = counter[device];
  }
  const int ctas = n >= 64 * 512 ? kArgmaxCtas : 1;
  return op_launch(argmax_advance_kernel, dim3(ctas), 512, 0, stream, logits_dev, n, tok_dev, pos_dev, history_dev, forced_dev,
                   history_cap, pv, pi, cnt);
}

GOPH_API int goph_mlx_embed(float* out_dev, uint64_t out_len, const goph_mlx_weight* w, const int* tok_dev, void* stream) {
  clear_error();
  if (!w || w->magic != kMagicMLX) return fail(GOPH_E_INVALID, "invalid MLX weight handle");
  if (!out_dev || out_len < (uint64_t)w->in_dim || !tok_dev) return fail(GOPH_E_INVALID, "goph_mlx_embed: buffers");
  if (int rc = use_device(w->device)) return rc;
  const int words = w->in_dim / 8;
  return op_launch(embed_mlx_kernel, dim3((words + 127) / 128), 128, 0, stream, out_dev, (const uint32_t*)w->qweight,
                   (const void*)w->sb, (const unsigned char*)w->tiled, tok_dev, w->in_dim, w->group_size, w->sb_bf16);
}
