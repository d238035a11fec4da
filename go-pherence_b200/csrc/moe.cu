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
// The steps of a call, whatever the number of tokens; nothing returns to the host:
//   1. router logits     — moe_router_kernel, or the MLX GEMM kernel for a router in the tiled layout
//   2. moe_route_kernel  — one CTA per token does the softmax/top-k in the reference's order; the
//      last CTA to finish then groups the (token, slot) items by expert: the list of experts that
//      were selected at all and, per expert, its items; for experts in the tiled layout also work
//      entries of up to 2 or 4 items.  (1 and 2 are one launch, moe_router_route_kernel, for a
//      row-major router of up to 128 experts.)
//   3. gate and up — row-major experts: moe_expert_kernel<phase 0>, grid (row blocks, selected
//      experts): a warp streams row r of the expert's gate and up matrices ONCE and applies it to up
//      to four of the expert's tokens at a time (their x staged in shared memory), writing
//      silu(g) * u per item.  Tiled experts: the entries' activations as digits
//      (moe_mma_prep_kernel), then one grouped launch of the tensor-core GEMV kernel over the
//      (entry, matrix, 128-row tile) items (mlx_mma.cu)
//   4. down — the same two forms, writing one vector per item
//   5. moe_combine_kernel — out[t] = sum over the token's slots, in selection order, of
//      weight * vector, so the result does not depend on scheduling.
// One token on row-major experts: all five steps as phases of one cooperative launch (moe_token_kernel).
// Each expert matrix is read from HBM once per call however many tokens chose the expert.
// Experts that are not resident on this GPU (multi-GPU placement) are skipped: the output is then
// this GPU's partial sum.
#include <string.h>

#include <mutex>
#include <vector>

#include "goph_internal.cuh"
#include "mlx_mma.cuh"
#include "tc_common.cuh"

namespace goph {

constexpr uint32_t kMagicMoE = 0x4d4f4558;  // "MOEX"
constexpr int kMoeWarps = 8, kMoeThreads = kMoeWarps * 32;
constexpr int kMoeDepth = 4;             // steps of a warp's weight ring
constexpr int kMoeStepBytes = 1024 + 512;  // two rows x 32 lanes x 16 B of weights, two rows x 32 lanes x 8 B of scales
constexpr int kMoeMaxExperts = 1024;
constexpr int kMoeMaxTopK = 64;      // slots of a token the one-launch form keeps in shared memory  // the routing kernel keeps one float and one int per expert in shared memory

struct MoeTables {
  const uint4** gate_w;   // [E] packed rows (16-byte units) or null when the expert is not resident
  const void** gate_sb;   // [E] {scale,bias} table
  const uint4** up_w;
  const void** up_sb;
  const uint4** down_w;
  const void** down_sb;
};

// One selected, resident expert of the current call.
struct __align__(16) MoeWork {
  const uint4* w[3];   // gate, up, down rows
  const void* sb[3];
  int expert, count;   // count = items (token, slot) that chose it
  int pad[2];
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
  int* lists;                      // [0] arrival counter of the routing CTAs, [1] number of work entries
  goph::MoeWork* work;             // [E] selected resident experts of the current call
  int* items;                      // [E][max_tokens] item = token * top_k + slot, per expert
  // experts in the tiled layout: grouped launches of the tensor-core kernel
  int tiled;                       // -1 no expert set yet, 0 row-major experts, 1 tiled experts
  int max_entries;                 // work entries (expert, up to two items) a call can have
  goph::MmaGroupEntry* mwork;      // [max_entries]
  unsigned char* mxb;              // [max_entries] prepared activations of an entry
  float* mxtab;                    // [max_entries] their sums and scales
  float* gu;                       // [max_entries * 2][2][inter] gate and up results (entries of two or four items: the first holds more entries)
  // one token, row-major experts: the whole call as one cooperative launch
  unsigned* bar;                   // [0] barrier counter (only grows), [1] its value when the next launch starts, [2] set when a wait gave up
  int token_grid;                  // CTAs of that launch (0 = not asked yet, -1 = does not fit)
  int no_router_cluster;           // set when the device refused the router + routing cluster launch
  size_t token_smem;
};

// The layers alive on each device: clearing the device's status also resets their barrier words.
static std::mutex g_layers_mu;
static std::vector<goph_moe_layer*> g_layers;


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

__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// The router rows of one block of 16 experts against token t: a CTA stages the token's x and each
// warp takes two expert rows.  `wait` is called once, after the first weights are in flight and
// before x is read (the caller's dependency on the kernel in front).
template <bool SB_BF16, typename Wait>
__device__ __forceinline__ void moe_router_block(const uint4* __restrict__ w, const void* __restrict__ sb,
                                                 const float* __restrict__ x, float* __restrict__ logits, int num_experts,
                                                 int hidden, int ug_shift, int groups, int eblock, int t,
                                                 unsigned char* smem_raw, Wait wait) {
  const int units = hidden / 32, iters = (units + 31) / 32;
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)iters * 256 * 16);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e0 = (eblock * kMoeWarps + warp) * 2, e1 = min(e0 + 1, num_experts - 1);
  const size_t sb_row = (size_t)groups * (SB_BF16 ? 4 : 8);
  // the weights do not depend on the kernel in front: first units in flight before the wait
  uint4 q[2];
  const bool live = e0 < num_experts;
  const int u0 = min(lane, units - 1);
  if (live) {
    q[0] = ld_stream(w + (size_t)e0 * units + u0);
    q[1] = ld_stream(w + (size_t)e1 * units + u0);
  }
  wait();
  for (int idx = threadIdx.x; idx < iters * 256; idx += kMoeThreads) {
    const int it = idx >> 8, slot = (idx >> 5) & 7, l = idx & 31, unit = it * 32 + l;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (unit < units) v = *reinterpret_cast<const float4*>(x + (size_t)t * hidden + (size_t)unit * 32 + slot * 4);
    xs[idx] = v;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < iters * 32; idx += kMoeThreads) {
    const int it = idx >> 5, l = idx & 31;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float4 v = xs[(it * 8 + k) * 32 + l];
      s += (v.x + v.y) + (v.z + v.w);
    }
    xc[idx] = make_float2(16.f * s, s);
  }
  __syncthreads();
  if (!live) return;
  float acc[2] = {0.f, 0.f};
  for (int it = 0; it < iters; ++it) {
    int unit = it * 32 + lane;
    const bool valid = unit < units;
    if (!valid) unit = units - 1;
    uint4 nq[2] = {q[0], q[1]};
    if (it + 1 < iters) {
      const int nu = min((it + 1) * 32 + lane, units - 1);
      nq[0] = ld_stream(w + (size_t)e0 * units + nu);
      nq[1] = ld_stream(w + (size_t)e1 * units + nu);
    }
    const int grp = unit >> ug_shift;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int e = r ? e1 : e0;
      float sc, bi;
      if (SB_BF16) {
        uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(sb) + e * sb_row) + grp);
        sc = __uint_as_float(v << 16);
        bi = __uint_as_float(v & 0xFFFF0000u);
      } else {
        float2 v = __ldg(reinterpret_cast<const float2*>(reinterpret_cast<const char*>(sb) + e * sb_row) + grp);
        sc = v.x;
        bi = v.y;
      }
      float2 F = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t word = k == 0 ? q[r].x : k == 1 ? q[r].y : k == 2 ? q[r].z : q[r].w;
        float f[8];
        unpack16(word, f);
        const float4 xa = xs[(it * 8 + 2 * k) * 32 + lane], xb = xs[(it * 8 + 2 * k + 1) * 32 + lane];
        fma2(F, make_float2(f[0], f[1]), make_float2(xa.x, xa.y));
        fma2(F, make_float2(f[2], f[3]), make_float2(xa.z, xa.w));
        fma2(F, make_float2(f[4], f[5]), make_float2(xb.x, xb.y));
        fma2(F, make_float2(f[6], f[7]), make_float2(xb.z, xb.w));
      }
      const float2 c = xc[it * 32 + lane];
      if (valid) {
        acc[r] = fmaf(sc, (F.x + F.y) - c.x, acc[r]);
        acc[r] = fmaf(bi, c.y, acc[r]);
      }
    }
    q[0] = nq[0];
    q[1] = nq[1];
  }
  const float a0 = warp_sum(acc[0]), a1 = warp_sum(acc[1]);
  if (lane == 0) {
    logits[(size_t)t * num_experts + e0] = a0;
    if (e0 + 1 < num_experts) logits[(size_t)t * num_experts + e0 + 1] = a1;
  }
}

// Router logits for every token in one launch: grid (expert blocks of 16, tokens).  (The batched MLX
// kernel would run ceil(T/8) launches over the same small matrix.)
template <bool SB_BF16>
__global__ void __launch_bounds__(kMoeThreads)
moe_router_kernel(const uint4* __restrict__ w, const void* __restrict__ sb, const float* __restrict__ x,
                  float* __restrict__ logits, int num_experts, int hidden, int ug_shift, int groups) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  moe_router_block<SB_BF16>(w, sb, x, logits, num_experts, hidden, ug_shift, groups, blockIdx.x, blockIdx.y, smem_raw,
                            [] { asm volatile("griddepcontrol.wait;" ::: "memory"); });
}

// simd.SoftmaxInPlace + the top-k loop of moeForwardWithREAP in the reference's order
// (model/moe.go:226-280; backends/simd/runtime/softmax.go:9-30): one CTA per token; the
// exponentials are taken in parallel, the sum by one thread in index order, the k rounds of
// "largest probability not yet picked, lowest id on ties" by a warp over shared memory.  The last
// CTA to finish groups the (token, slot) items by expert into the work list.
// Tuning build only: CTA 1 records the clock at the phase boundaries of the one-launch form.
#ifdef GOPH_TUNING
__device__ long long g_moe_trace[24];
#define MTP(k) if (blockIdx.x == 1 && threadIdx.x == 0) g_moe_trace[k] = clock64();
#define RTP(k) if (blockIdx.x == 1 && threadIdx.x == 0) g_moe_trace[k] = clock64();
#else
#define MTP(k)
#define RTP(k)
#endif
struct MoeRouteShared {
  float sp[kMoeMaxExperts];
  float mx, inv;
  int ok;
};

// One token's routing by the calling CTA (any number of threads, at least one warp): softmax over the
// logits and the top-k rounds; ids (-1 = none) and weights go to my_ids / my_w (global or shared).
__device__ __forceinline__ void moe_route_token(const float* __restrict__ lg, int num_experts, int top_k, int norm_topk,
                                                int* my_ids, float* my_w, MoeRouteShared& sh) {
  const int tid = threadIdx.x, lane = tid & 31;
  float* sp = sh.sp;
  for (int i = tid; i < num_experts; i += blockDim.x) sp[i] = __ldcg(lg + i);
  __syncthreads();
  RTP(16)
  if (tid < 32) {
    float mx = -INFINITY;
    for (int i = lane; i < num_experts; i += 32) mx = fmaxf(mx, sp[i]);  // skips NaN, as "x > mx" does
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // the reference starts from x[0]: if that is NaN every comparison is false and the maximum stays NaN
    if (isnan(sp[0])) mx = sp[0];
    if (lane == 0) sh.mx = mx;
  }
  __syncthreads();
  RTP(17)
  for (int i = tid; i < num_experts; i += blockDim.x) sp[i] = (float)exp((double)(sp[i] - sh.mx));
  __syncthreads();
  RTP(18)
  if (tid == 0) {
    float sum = 0.f;
    // index order, one rounding per element; the loads of a batch are issued together
    for (int i0 = 0; i0 < num_experts; i0 += 16) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = i0 + j < num_experts ? sp[i0 + j] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (i0 + j < num_experts) sum = __fadd_rn(sum, v[j]);
    }
    sh.ok = !(sum == 0.f || isnan(sum) || isinf(sum));  // SoftmaxInPlace fails: no expert runs
    sh.inv = __fdiv_rn(1.f, sum);
  }
  __syncthreads();
  RTP(19)
  if (sh.ok)
    for (int i = tid; i < num_experts; i += blockDim.x) sp[i] = __fmul_rn(sp[i], sh.inv);
  __syncthreads();
  RTP(20)
  if (tid < 32 && num_experts <= 128 && top_k <= 32) {
    // The usual sizes: a lane keeps its four candidates in registers over the rounds, lane k keeps
    // the k-th pick, and the picks are normalised and stored by their lanes at the end.  Same picks
    // (largest probability, lowest id on ties) and the same additions, in the same order, as the
    // general form below.
    // A probability p >= 0 becomes the key bits(p) + 1, which orders as p does; 0 marks "none" or
    // "already picked".  A round = the largest key of the warp, then the lowest index that holds it.
    uint32_t key[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p = lane + 32 * i < num_experts ? sp[lane + 32 * i] : -1.f;
      key[i] = p >= 0.f ? __float_as_uint(p) + 1u : 0u;  // a NaN cannot be here: the sum would have failed
    }
    int n = 0, sel_id = -1;
    float wsum = 0.f, sel_w = 0.f;
    const bool ok = sh.ok != 0;
    for (int k = 0; k < top_k && ok; ++k) {
      uint32_t mine = 0u;
      int at = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (key[i] > mine) {
          mine = key[i];
          at = i;
        }
      }
      const uint32_t top = __reduce_max_sync(0xffffffffu, mine);
      if (top == 0u) break;  // nothing left to pick, in this round and after it
      const int best = (int)__reduce_min_sync(0xffffffffu, mine == top ? (uint32_t)(lane + 32 * at) : 0x7fffffffu);
      const float bs = __uint_as_float(top - 1u);
      if (lane == n) {
        sel_id = best;
        sel_w = bs;
      }
      if ((best & 31) == lane) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if ((best >> 5) == i) key[i] = 0u;
      }
      wsum = __fadd_rn(wsum, bs);
      ++n;
    }
    if (lane < top_k) {
      const bool have = lane < n;
      float w = have ? sel_w : 0.f;
      if (have && norm_topk && wsum > 0.f) w = __fdiv_rn(w, wsum);
      my_ids[lane] = have ? sel_id : -1;
      my_w[lane] = w;
    }
  } else if (tid < 32) {
    int n = 0;
    float wsum = 0.f;
    for (int k = 0; k < top_k; ++k) {
      int best = -1;
      float bs = -1.f;  // probabilities are >= 0; a picked entry is overwritten with -2 and never wins again
      if (sh.ok) {
        for (int j = lane; j < num_experts; j += 32) {
          float v = sp[j];
          if (v > bs) {
            best = j;
            bs = v;
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
          sp[best] = -2.f;
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
    }
  }
}

struct MoeRouteArgs {
  const float* logits;
  int num_experts, top_k, norm_topk, tokens, max_tokens;
  MoeTables tb;
  int* ids;
  float* wts;
  int* lists;
  MoeWork* work;
  int* items;
  MmaGroupEntry* mwork;
  int max_entries, entry_rows;
};

// Token t's routing by the calling CTA; the CTA that finishes the call's last token then groups the
// (token, slot) items by expert into the work lists.
__device__ __forceinline__ void moe_route_body(const MoeRouteArgs& ra, int t) {
  __shared__ MoeRouteShared sh;
  __shared__ int s_cnt[kMoeMaxExperts];
  __shared__ int s_last, s_n, s_m;
  const float* logits = ra.logits;
  const int num_experts = ra.num_experts, top_k = ra.top_k, norm_topk = ra.norm_topk, tokens = ra.tokens;
  const int max_tokens = ra.max_tokens, max_entries = ra.max_entries, entry_rows = ra.entry_rows;
  const MoeTables& tb = ra.tb;
  int* ids = ra.ids;
  float* wts = ra.wts;
  int* lists = ra.lists;
  MoeWork* work = ra.work;
  int* items = ra.items;
  MmaGroupEntry* mwork = ra.mwork;
  const int tid = threadIdx.x;
  moe_route_token(logits + (size_t)t * num_experts, num_experts, top_k, norm_topk, ids + (size_t)t * top_k,
                  wts + (size_t)t * top_k, sh);
  if (tid == 0) {
    if (tokens > 1) {
      __threadfence();
      s_last = atomicAdd(&lists[0], 1) == tokens - 1;
    } else {
      s_last = 1;  // the only CTA builds the work list itself
    }
  }
  __syncthreads();
  if (!s_last) return;
  // ---- last CTA: group the items by expert.  The order inside a list and of the work entries
  // depends on scheduling; no result does (every item's arithmetic is the same in any grouping).
  __threadfence();
  for (int e = tid; e < num_experts; e += blockDim.x) s_cnt[e] = 0;
  if (tid == 0) s_n = s_m = 0;
  __syncthreads();
  for (int it = tid; it < tokens * top_k; it += blockDim.x) {
    const int e = __ldcg(ids + it);
    if (e >= 0 && tb.gate_w[e] != nullptr) items[(size_t)e * max_tokens + atomicAdd(&s_cnt[e], 1)] = it;
  }
  __syncthreads();
  for (int e = tid; e < num_experts; e += blockDim.x) {
    if (s_cnt[e] > 0) {
      MoeWork wk;
      wk.w[0] = tb.gate_w[e];
      wk.w[1] = tb.up_w[e];
      wk.w[2] = tb.down_w[e];
      wk.sb[0] = tb.gate_sb[e];
      wk.sb[1] = tb.up_sb[e];
      wk.sb[2] = tb.down_sb[e];
      wk.expert = e;
      wk.count = s_cnt[e];
      wk.pad[0] = wk.pad[1] = 0;
      work[atomicAdd(&s_n, 1)] = wk;
      if (mwork) {
        // tiled experts: entries of up to entry_rows items, an expert's entries next to each other
        const int n = (s_cnt[e] + entry_rows - 1) / entry_rows;
        const int first = atomicAdd(&s_m, n);
        for (int j = 0; j < n && first + j < max_entries; ++j) {
          MmaGroupEntry ge;
          ge.w[0] = reinterpret_cast<const unsigned char*>(tb.gate_w[e]);
          ge.w[1] = reinterpret_cast<const unsigned char*>(tb.up_w[e]);
          ge.w[2] = reinterpret_cast<const unsigned char*>(tb.down_w[e]);
          ge.expert = e;
          ge.count = min(entry_rows, s_cnt[e] - j * entry_rows);
          for (int q = 0; q < 8; ++q) ge.item[q] = q < ge.count ? items[(size_t)e * max_tokens + j * entry_rows + q] : 0;
          mwork[first + j] = ge;
        }
      }
    }
  }
  __syncthreads();
  // entries past the selected experts: count 0 tells their CTAs to return
  for (int y = s_n + tid; y < num_experts; y += blockDim.x) work[y].count = 0;
  if (tid == 0) {
    lists[1] = s_n;
    lists[2] = min(s_m, max_entries);
    lists[0] = 0;  // ready for the next call
  }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const __grid_constant__ MoeRouteArgs ra) {
  pdl_prologue();
  moe_route_body(ra, blockIdx.x);
}

// Router rows and routing in one launch: the CTAs of a token (one per block of 16 experts, at most 8)
// form a thread-block cluster; each computes its experts' logits, the cluster meets (which orders
// the logits it wrote), and its first CTA routes the token.
template <bool SB_BF16>
__global__ void __launch_bounds__(kMoeThreads)
moe_router_route_kernel(const uint4* __restrict__ w, const void* __restrict__ sb, const float* __restrict__ x,
                        float* __restrict__ logits, int hidden, int ug_shift, int groups, int cs,
                        const __grid_constant__ MoeRouteArgs ra) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int t = blockIdx.x / cs, rank = blockIdx.x - t * cs;
  moe_router_block<SB_BF16>(w, sb, x, logits, ra.num_experts, hidden, ug_shift, groups, rank, t, smem_raw,
                            [] { asm volatile("griddepcontrol.wait;" ::: "memory"); });
  tc::cluster_sync_all();
  if (rank != 0) return;
  moe_route_body(ra, t);
}

// Sums N values over the warp with N-1 + 5-log2(N) shuffles: at each of the first log2(N) butterfly
// steps a lane keeps one half of its values and hands the other half to its partner.  Every value is
// added in the same lane pairs as a plain xor butterfly, so the result does not depend on N.
// On return v[0] is the total of value number idx(lane), idx = the lane's bits 4,3,.. read as a number.
template <int N>
__device__ __forceinline__ void warp_sum_split(float (&v)[N], int lane) {
  int o = 16;
#pragma unroll
  for (int n = N; n > 1; n >>= 1, o >>= 1) {
    const bool upper = lane & o;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      float keep = upper ? v[i + n / 2] : v[i];
      float give = upper ? v[i] : v[i + n / 2];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, give, o);
    }
  }
  for (; o; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
}

// The expert kernels.  PHASE 0: rows of gate and up (one row of each per warp task) against the
// expert's tokens' x, writing silu(g) * u per item; PHASE 1: two adjacent rows of down per task against
// the items' activations, writing one vector per item.  grid = (row blocks, work entries); a CTA
// walks its expert's items M at a time: vectors staged in shared memory as [vector][iteration][slot][lane]
// float4 plus {16*sum, sum} per 32-element unit, each packed word unpacked once and used M times, the
// next 16-byte units in flight while the current ones are computed.
template <bool SB_BF16, int PHASE, int M>
__device__ __forceinline__ void moe_expert_pass(const MoeWork& wk, const int* __restrict__ items, int base, int m_now,
                                                const float* __restrict__ src, float* __restrict__ dst, int in_dim,
                                                int out_rows, int top_k, int ug_shift, int groups, float4* xs, float2* xc,
                                                unsigned char* ring, int bx, int nbx) {
  // bx of nbx: this CTA's place among the CTAs that share the expert's rows
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int units = in_dim / 32, iters = (units + 31) / 32;
  const size_t sb_row = (size_t)groups * (SB_BF16 ? 4 : 8);
  const int tasks = PHASE == 0 ? out_rows : (out_rows + 1) / 2;
  const int task_stride = nbx * kMoeWarps;
  struct Rows {
    const uint4* w[2];
    const char* sb[2];
    int row;
  };
  auto open_task = [&](int task, Rows& t) {
    if (PHASE == 0) {
      t.row = task;
      t.w[0] = wk.w[0] + (size_t)task * units;
      t.w[1] = wk.w[1] + (size_t)task * units;
      t.sb[0] = reinterpret_cast<const char*>(wk.sb[0]) + task * sb_row;
      t.sb[1] = reinterpret_cast<const char*>(wk.sb[1]) + task * sb_row;
    } else {
      t.row = task * 2;
      const int r1 = min(t.row + 1, out_rows - 1);
      t.w[0] = wk.w[2] + (size_t)t.row * units;
      t.w[1] = wk.w[2] + (size_t)r1 * units;
      t.sb[0] = reinterpret_cast<const char*>(wk.sb[2]) + t.row * sb_row;
      t.sb[1] = reinterpret_cast<const char*>(wk.sb[2]) + r1 * sb_row;
    }
  };
  // Per-warp ring of kMoeDepth steps in shared memory, filled with cp.async: a lane copies the 16-byte
  // unit and the {scale,bias} entry it will itself consume, so completion of the lane's own copy
  // group is all the synchronisation a step needs, and kMoeDepth - 1 steps of every warp are in
  // flight while one is computed.  A step = one 32-lane iteration over the two rows of a task.
  unsigned char* wring = ring + (size_t)warp * kMoeDepth * kMoeStepBytes;
  int task = bx * kMoeWarps + warp;
  const int my_tasks = task < tasks ? (tasks - task + task_stride - 1) / task_stride : 0;
  const int nsteps = my_tasks * iters;
  auto issue = [&](int q) {
    if (q < nsteps) {
      const int j = q / iters, it = q - j * iters;
      Rows t;
      open_task(task + j * task_stride, t);
      int unit = it * 32 + lane;
      if (unit >= units) unit = units - 1;  // the staged vector is zero there
      const int grp = unit >> ug_shift;
      unsigned char* slot = wring + (size_t)(q % kMoeDepth) * kMoeStepBytes;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint32_t dw = (uint32_t)__cvta_generic_to_shared(slot + r * 512 + lane * 16);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dw), "l"(t.w[r] + unit) : "memory");
        const uint32_t ds = (uint32_t)__cvta_generic_to_shared(slot + 1024 + r * 256 + lane * 8);
        if (SB_BF16)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(ds), "l"(reinterpret_cast<const uint32_t*>(t.sb[r]) + grp) : "memory");
        else
          asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(ds), "l"(reinterpret_cast<const float2*>(t.sb[r]) + grp) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // one group per step, empty past the end
  };
#pragma unroll
  for (int q = 0; q < kMoeDepth - 1; ++q) issue(q);  // first weights in flight while the vectors are staged
  // ---- stage the m_now vectors -----------------------------------------------------------
  const int per_m = iters * 256;
  for (int idx = threadIdx.x; idx < M * per_m; idx += kMoeThreads) {
    const int m = idx / per_m, rem = idx - m * per_m;
    const int it = rem >> 8, slot = (rem >> 5) & 7, l = rem & 31, unit = it * 32 + l;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m < m_now && unit < units) {
      const int item = items[base + m];
      const float* p = src + (size_t)(PHASE == 0 ? item / top_k : item) * in_dim + (size_t)unit * 32 + slot * 4;
      v = *reinterpret_cast<const float4*>(p);
    }
    xs[idx] = v;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < M * iters * 32; idx += kMoeThreads) {
    const int mi = idx >> 5, l = idx & 31;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float4 v = xs[(mi * 8 + k) * 32 + l];
      s += (v.x + v.y) + (v.z + v.w);
    }
    xc[idx] = make_float2(16.f * s, s);
  }
  __syncthreads();

  float acc[2][M];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
  Rows cur_rows;
  for (int q = 0; q < nsteps; ++q) {
    const int j = q / iters, it = q - j * iters;
    if (it == 0) open_task(task + j * task_stride, cur_rows);
    issue(q + kMoeDepth - 1);
    asm volatile("cp.async.wait_group %0;" ::"n"(kMoeDepth - 1) : "memory");
    const unsigned char* slot = wring + (size_t)(q % kMoeDepth) * kMoeStepBytes;
    uint4 cw[2];
    uint32_t cs[2], cb[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      cw[r] = *reinterpret_cast<const uint4*>(slot + r * 512 + lane * 16);
      if (SB_BF16) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(slot + 1024 + r * 256 + lane * 8);
        cs[r] = v << 16;
        cb[r] = v & 0xFFFF0000u;
      } else {
        const float2 v = *reinterpret_cast<const float2*>(slot + 1024 + r * 256 + lane * 8);
        cs[r] = __float_as_uint(v.x);
        cb[r] = __float_as_uint(v.y);
      }
    }
    {
      float2 F[2][M];
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) F[r][m] = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float4 xa[M], xb[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4* bp = xs + ((size_t)(m * iters + it) * 8 + 2 * k) * 32 + lane;
          xa[m] = bp[0];
          xb[m] = bp[32];
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint32_t word = k == 0 ? cw[r].x : k == 1 ? cw[r].y : k == 2 ? cw[r].z : cw[r].w;
          float f[8];
          unpack16(word, f);
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
        const float2 c = xc[(m * iters + it) * 32 + lane];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float dot = (F[r][m].x + F[r][m].y) - c.x;
          acc[r][m] = fmaf(__uint_as_float(cs[r]), dot, acc[r][m]);
          acc[r][m] = fmaf(__uint_as_float(cb[r]), c.y, acc[r][m]);
        }
      }
    }
    if (it != iters - 1) continue;
    // ---- reduce the 2*M sums; value number 2*m + r ends up in the lanes whose top bits spell it
    float v[2 * M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      v[2 * m] = acc[0][m];
      v[2 * m + 1] = acc[1][m];
      acc[0][m] = acc[1][m] = 0.f;
    }
    warp_sum_split<2 * M>(v, lane);
    constexpr int kLow = 16 / M;              // lane bit that tells row 0 from row 1
    const int m_of_lane = lane / (2 * kLow);  // lane bits above kLow
    const int r_of_lane = (lane / kLow) & 1;
    const float mine = v[0];
    const float other = __shfl_xor_sync(0xffffffffu, mine, kLow);
    if ((lane & (kLow - 1)) == 0 && m_of_lane < m_now) {
      const int item = items[base + m_of_lane];
      if (PHASE == 0) {
        if (r_of_lane == 0) {
          // kernels.SiLU then the multiply (backends/simd/kernels/activation.go:15-24)
          // single-precision exp (2 ulp) where the reference rounds an f64 exp: the FP64 pipe is slow
          const float sv = __fdiv_rn(mine, __fadd_rn(1.0f, expf(-mine)));
          dst[(size_t)item * out_rows + cur_rows.row] = __fmul_rn(sv, other);
        }
      } else {
        const int row = cur_rows.row + r_of_lane;
        if (row < out_rows) dst[(size_t)item * out_rows + row] = mine;
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
}

template <bool SB_BF16, int PHASE>
__global__ void __launch_bounds__(kMoeThreads, 2)
moe_expert_kernel(const MoeWork* __restrict__ work, const int* __restrict__ lists, const int* __restrict__ items_all,
                  const float* __restrict__ src, float* __restrict__ dst, int max_tokens, int in_dim, int out_rows,
                  int top_k, int ug_shift, int groups) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_prologue();
  const MoeWork wk = work[blockIdx.y];  // entries past the selected experts carry count 0
  if (wk.count == 0) return;
  const int* items = items_all + (size_t)wk.expert * max_tokens;
  const int iters = (in_dim / 32 + 31) / 32;
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  unsigned char* ring = smem_raw + (size_t)4 * iters * (256 * 16 + 32 * 8);  // behind room for four vectors
  // M vectors per pass: 1, 2 or 4 by how many items the expert has
  if (wk.count == 1) {
    float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)1 * iters * 256 * 16);
    moe_expert_pass<SB_BF16, PHASE, 1>(wk, items, 0, 1, src, dst, in_dim, out_rows, top_k, ug_shift, groups, xs, xc, ring,
                                       blockIdx.x, gridDim.x);
  } else if (wk.count == 2) {
    float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)2 * iters * 256 * 16);
    moe_expert_pass<SB_BF16, PHASE, 2>(wk, items, 0, 2, src, dst, in_dim, out_rows, top_k, ug_shift, groups, xs, xc, ring,
                                       blockIdx.x, gridDim.x);
  } else {
    float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)4 * iters * 256 * 16);
    for (int base = 0; base < wk.count; base += 4) {
      if (base) __syncthreads();
      moe_expert_pass<SB_BF16, PHASE, 4>(wk, items, base, min(4, wk.count - base), src, dst, in_dim, out_rows, top_k,
                                         ug_shift, groups, xs, xc, ring, blockIdx.x, gridDim.x);
    }
  }
}

// out[t][r] = sum over slots k in selection order of weight[t][k] * dpart[t][k][r]
// (out[i] += weight * down[i], model/moe.go:336-344).  Slots whose expert is not resident here add nothing.
__device__ __forceinline__ float moe_combine_row(const MoeTables& tb, const float* __restrict__ dpart,
                                                 const int* __restrict__ ids, const float* __restrict__ wts, int t, int r,
                                                 int hidden, int top_k) {
  float acc = 0.f;
  for (int k0 = 0; k0 < top_k; k0 += 8) {  // eight slots at a time: their loads are issued together
    int e[8];
    float w[8], d[8];
    bool on[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = k0 + j < top_k ? ids[t * top_k + k0 + j] : -1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      on[j] = e[j] >= 0 && tb.down_w[e[j]] != nullptr;
      w[j] = on[j] ? wts[t * top_k + k0 + j] : 0.f;
      d[j] = on[j] ? __ldcg(dpart + ((size_t)t * top_k + k0 + j) * hidden + r) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (on[j]) acc = __fadd_rn(acc, __fmul_rn(w[j], d[j]));
  }
  return acc;
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(MoeTables tb, const float* __restrict__ dpart, const int* __restrict__ ids,
                   const float* __restrict__ wts, float* __restrict__ out, int hidden, int top_k) {
  pdl_prologue();
  const int t = blockIdx.y;
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= hidden) return;
  out[(size_t)t * hidden + r] = moe_combine_row(tb, dpart, ids, wts, t, r, hidden, top_k);
}

// One token, one launch: router rows, routing, gate and up, down and the weighted sum as phases of
// one cooperative kernel (every CTA resident) with a grid-wide barrier where a phase reads what
// another CTA wrote.  Each phase runs the code of the kernel it replaces on the same operands, so
// the result has the bits of the five-launch form.  The barrier: a device counter that only grows
// (one releasing add per CTA, one polling thread per CTA, bounded; a wait that runs out records
// 700 + the barrier's number in the status word and the CTA returns).
constexpr long long kMoeBarrierTimeoutCycles = 2000000000LL;  // about a second
template <bool RSB_BF16, bool SB_BF16>
__global__ void __launch_bounds__(kMoeThreads, 2)
moe_token_kernel(MoeTables tb, const uint4* __restrict__ rw, const void* __restrict__ rsb, int r_shift, int r_groups,
                 const float* __restrict__ x, const float* __restrict__ logits_in, float* __restrict__ logits,
                 int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ act, float* __restrict__ dpart,
                 float* __restrict__ out, unsigned* __restrict__ bar, int* __restrict__ status, int num_experts,
                 int hidden, int inter, int top_k, int norm_topk, int ug_shift, int group_size) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ MoeRouteShared sh;
  __shared__ int s_ids[kMoeMaxTopK];
  __shared__ float s_wts[kMoeMaxTopK];
  __shared__ unsigned s_base;
  __shared__ int s_abort;
  MTP(0)
  pdl_prologue();
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_base = *reinterpret_cast<volatile unsigned*>(bar + 1);
    // a launch whose wait gave up leaves the counter between two launches' values: every later
    // launch returns at once (status already set) until goph_kernel_status_clear resets the words
    s_abort = *reinterpret_cast<volatile unsigned*>(bar + 2) != 0u;
  }
  __syncthreads();
  if (s_abort) return;
  int nbar = 0;
  auto grid_barrier = [&]() {
    __syncthreads();
    ++nbar;
    if (tid == 0) {
      asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(bar), "r"(1u) : "memory");
      const unsigned target = s_base + (unsigned)nbar * gridDim.x;
      const long long t0 = clock64();
      unsigned seen;
      while (true) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(bar) : "memory");
        if ((int)(seen - target) >= 0) break;
        if (clock64() - t0 > kMoeBarrierTimeoutCycles) {
          s_abort = 1;
          atomicExch(status, 700 + nbar);
          atomicExch(bar + 2, 1u);
          break;
        }
      }
    }
    __syncthreads();
    return s_abort == 0;
  };
  // ---- router rows (unless the caller supplied the logits) ----
  const float* lg = logits_in;
  if (!lg) {
    if ((int)blockIdx.x * 2 * kMoeWarps < num_experts)
      moe_router_block<RSB_BF16>(rw, rsb, x, logits, num_experts, hidden, r_shift, r_groups, blockIdx.x, 0, smem_raw, [] {});
    MTP(1)
    if (!grid_barrier()) return;
    MTP(2)
    lg = logits;
  }
  // ---- routing, by every CTA for itself ----
  moe_route_token(lg, num_experts, top_k, norm_topk, s_ids, s_wts, sh);
  __syncthreads();
  MTP(3)
  if (blockIdx.x == 0 && tid < top_k) {
    ids[tid] = s_ids[tid];
    wts[tid] = s_wts[tid];
  }
  // ---- gate and up, then down: CTA b works for slot b % top_k with the CTAs b' = b (mod top_k) ----
  const int slot = blockIdx.x % top_k, bx = blockIdx.x / top_k, nbx = gridDim.x / top_k;
  const int e = s_ids[slot];
  const bool mine = bx < nbx && e >= 0 && tb.gate_w[e] != nullptr;
  MoeWork wk;
  if (mine) {
    wk.w[0] = tb.gate_w[e];
    wk.w[1] = tb.up_w[e];
    wk.w[2] = tb.down_w[e];
    wk.sb[0] = tb.gate_sb[e];
    wk.sb[1] = tb.up_sb[e];
    wk.sb[2] = tb.down_sb[e];
  }
  wk.expert = e;
  wk.count = 1;
  __shared__ int s_item;
  if (tid == 0) s_item = slot;  // item = token * top_k + slot, token 0
  __syncthreads();
  const int big = hidden > inter ? hidden : inter, iters_max = (big / 32 + 31) / 32;
  unsigned char* ring = smem_raw + (size_t)iters_max * (256 * 16 + 32 * 8);
  float4* xs = reinterpret_cast<float4*>(smem_raw);
  for (int phase = 0; phase < 2; ++phase) {
    const int in_dim = phase == 0 ? hidden : inter, out_rows = phase == 0 ? inter : hidden;
    const int iters = (in_dim / 32 + 31) / 32;
    float2* xc = reinterpret_cast<float2*>(smem_raw + (size_t)iters * 256 * 16);
    if (mine) {
      if (phase == 0)
        moe_expert_pass<SB_BF16, 0, 1>(wk, &s_item, 0, 1, x, act, in_dim, out_rows, top_k, ug_shift, in_dim / group_size, xs, xc,
                                       ring, bx, nbx);
      else
        moe_expert_pass<SB_BF16, 1, 1>(wk, &s_item, 0, 1, act, dpart, in_dim, out_rows, top_k, ug_shift, in_dim / group_size, xs,
                                       xc, ring, bx, nbx);
    }
    MTP(4 + 2 * phase)
    if (!grid_barrier()) return;
    MTP(5 + 2 * phase)
  }
  // ---- the weighted sum of the slots' vectors, in selection order ----
  for (int r = blockIdx.x * kMoeThreads + tid; r < hidden; r += gridDim.x * kMoeThreads)
    out[r] = moe_combine_row(tb, dpart, s_ids, s_wts, 0, r, hidden, top_k);
  // the counter's value when the next launch starts (every CTA has read the old one: all of them
  // passed the barriers above)
  if (blockIdx.x == 0 && tid == 0) bar[1] = s_base + (unsigned)nbar * gridDim.x;
  MTP(8)
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
  note_launch();
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
  if (num_experts > kMoeMaxExperts) return fail(GOPH_E_UNSUPPORTED, "MoE: at most %d experts per layer, got %d", kMoeMaxExperts, num_experts);
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
  m->tiled = -1;
  m->max_entries = min(max_tokens * top_k, num_experts * ((max_tokens + kMoeMmaRowsMin - 1) / kMoeMmaRowsMin));
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
  if (e == cudaSuccess) e = cudaMalloc(&m->bar, 4 * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemset(m->bar, 0, 4 * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMalloc(&m->lists, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(m->lists, 0, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(&m->work, (size_t)num_experts * sizeof(goph::MoeWork));
  if (e == cudaSuccess) e = cudaMalloc(&m->items, (size_t)num_experts * max_tokens * sizeof(int));
  if (e != cudaSuccess) {
    int rc = fail_cuda(e, "cudaMalloc(MoE layer)");
    m->magic = 0;  // partial allocations are released by the process; the handle is not returned
    return rc;
  }
  m->tables_dirty = 1;
  {
    std::lock_guard<std::mutex> lock(g_layers_mu);
    g_layers.push_back(m);
  }
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
  const int tiled = gate && gate->tiled ? 1 : 0;
  for (int i = 0; i < 3; ++i) {
    const goph_mlx_weight* w = ws[i];
    if (!w || w->magic != kMagicMLX || w->device != m->device || w->out_dim != want_out[i] || w->in_dim != want_in[i] ||
        w->group_size != m->group_size)
      return fail(GOPH_E_INVALID, "expert %d: projection %d must be an MLX weight [%d x %d] with group size %d on device %d", eid, i,
                  want_out[i], want_in[i], m->group_size, m->device);
    if ((w->tiled != nullptr) != (tiled != 0) || (!tiled && (!w->qweight || !w->sb)))
      return fail(GOPH_E_UNSUPPORTED, "expert %d: its projections mix the row-major and the tiled layout", eid);
    if (m->tiled >= 0 && m->tiled != tiled)
      return fail(GOPH_E_UNSUPPORTED, "expert %d: the experts of a layer must share one layout (row-major or tiled)", eid);
    if (m->sb_bf16 >= 0 && m->sb_bf16 != w->sb_bf16)
      return fail(GOPH_E_UNSUPPORTED, "experts mix bf16-valued and f32 scale tables");
  }
  if (tiled && !mlx_mma_grouped_supported(m->hidden, m->inter))
    return fail(GOPH_E_UNSUPPORTED, "tiled experts need hidden=%d and inter=%d to be multiples of 256", m->hidden, m->inter);
  if (tiled && !m->mwork) {
    // scratch of the grouped launches, once per layer
    if (int rc = use_device(m->device)) return rc;
    // sized for entries of two items (the most entries) holding four items' data (the largest entries)
    const int big = max(m->hidden, m->inter);
    const size_t xb = mlx_mma_grouped_xb_bytes(big, kMoeMmaRowsMax);
    const size_t tab = (size_t)mlx_mma_grouped_tab_floats(big, kMoeMmaRowsMax);
    const size_t ne = (size_t)m->max_entries;
    MmaGroupEntry* mw = nullptr;
    unsigned char* mxb = nullptr;
    float *mxtab = nullptr, *gu = nullptr;
    cudaError_t e = cudaMalloc(&mw, ne * sizeof(MmaGroupEntry));
    if (e == cudaSuccess) e = cudaMalloc(&mxb, ne * xb);
    if (e == cudaSuccess) e = cudaMalloc(&mxtab, ne * tab * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&gu, ne * kMoeMmaRowsMax * 2 * m->inter * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(mxb, 0, ne * xb);  // rows past an entry's items are multiplied too (and ignored)
    if (e != cudaSuccess) {
      cudaFree(mw);
      cudaFree(mxb);
      cudaFree(mxtab);
      cudaFree(gu);
      return fail_cuda(e, "cudaMalloc(MoE grouped-launch scratch)");
    }
    m->mwork = mw;
    m->mxb = mxb;
    m->mxtab = mxtab;
    m->gu = gu;
  }
  m->tiled = tiled;
  m->sb_bf16 = gate->sb_bf16;
  if (tiled) {
    m->host.gate_w[eid] = reinterpret_cast<const uint4*>(gate->tiled);
    m->host.up_w[eid] = reinterpret_cast<const uint4*>(up->tiled);
    m->host.down_w[eid] = reinterpret_cast<const uint4*>(down->tiled);
    m->host.gate_sb[eid] = m->host.up_sb[eid] = m->host.down_sb[eid] = nullptr;
  } else {
    m->host.gate_w[eid] = reinterpret_cast<const uint4*>(gate->qweight);
    m->host.gate_sb[eid] = gate->sb;
    m->host.up_w[eid] = reinterpret_cast<const uint4*>(up->qweight);
    m->host.up_sb[eid] = up->sb;
    m->host.down_w[eid] = reinterpret_cast<const uint4*>(down->qweight);
    m->host.down_sb[eid] = down->sb;
  }
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
  cudaFree(m->work);
  cudaFree(m->items);
  {
    std::lock_guard<std::mutex> lock(g_layers_mu);
    for (size_t i = 0; i < g_layers.size(); ++i)
      if (g_layers[i] == m) {
        g_layers.erase(g_layers.begin() + i);
        break;
      }
  }
  cudaFree(m->bar);
  cudaFree(m->mwork);
  cudaFree(m->mxb);
  cudaFree(m->mxtab);
  cudaFree(m->gu);
  m->magic = 0;
  delete m;
  return GOPH_OK;
}

static int* moe_status_word(int device) {
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

namespace goph {
int moe_status(int device) {
  int* p = moe_status_word(device);
  if (!p) return 0;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return v;
}
void moe_status_clear(int device) {
  int* p = moe_status_word(device);
  if (p) cudaMemset(p, 0, sizeof(int));
  std::lock_guard<std::mutex> lock(g_layers_mu);
  for (goph_moe_layer* m : g_layers)
    if (m->device == device) cudaMemset(m->bar, 0, 4 * sizeof(unsigned));
}
}  // namespace goph

typedef void (*MoeTokenKernel)(MoeTables, const uint4*, const void*, int, int, const float*, const float*, float*, int*, float*,
                               float*, float*, float*, unsigned*, int*, int, int, int, int, int, int, int);

// True when a call of one token can run as the one-launch form: row-major experts, a row-major
// router (or logits from the caller), option moe_fused on, and a device that holds the grid.
static bool moe_token_form(goph_moe_layer* m, const goph_mlx_weight* rw, MoeTokenKernel* kern) {
  if (!options().moe_fused || m->tiled != 0 || m->top_k > kMoeMaxTopK || m->token_grid < 0) return false;
  if (rw && !(rw->qweight && rw->sb && rw->group_size >= 32 && !(rw->group_size & (rw->group_size - 1)) && rw->in_dim % 32 == 0))
    return false;
  const bool rb = rw ? rw->sb_bf16 != 0 : true, eb = m->sb_bf16 != 0;
  *kern = rb ? (eb ? moe_token_kernel<true, true> : moe_token_kernel<true, false>)
             : (eb ? moe_token_kernel<false, true> : moe_token_kernel<false, false>);
  if (m->token_grid == 0) {
    const int big = max(m->hidden, m->inter), iters = (big / 32 + 31) / 32;
    const size_t smem = (size_t)iters * (256 * 16 + 32 * 8) + (size_t)kMoeWarps * kMoeDepth * kMoeStepBytes;
    int per_sm = 0;
    if (smem > (size_t)kSmemBudget || cudaFuncSetAttribute(*kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, *kern, kMoeThreads, smem) != cudaSuccess || per_sm < 1) {
      cudaGetLastError();
      m->token_grid = -1;
      return false;
    }
    if (per_sm > 2) per_sm = 2;
    const int grid = device_state(m->device).sm_count * per_sm;
    if (grid < m->top_k || grid * 2 * kMoeWarps < m->num_experts) {
      m->token_grid = -1;
      return false;
    }
    m->token_grid = grid;
    m->token_smem = smem;
  }
  return true;
}

// *declined: the launch was refused for lack of co-residency and nothing ran; the caller goes on with
// the other form.
static int moe_run_token(goph_moe_layer* m, MoeTokenKernel kern, float* out_dev, const float* x_dev, const goph_mlx_weight* rw,
                         const float* logits_dev, cudaStream_t s, bool* declined) {
  *declined = false;
  if (int rc = moe_upload_tables(m)) return rc;
  int* status = moe_status_word(m->device);
  if (!status) return fail(GOPH_E_NOMEM, "cannot allocate the MoE kernels' status word");
  int sh = 0, rsh = 0;
  while ((32 << sh) < m->group_size) ++sh;
  if (rw)
    while ((32 << rsh) < rw->group_size) ++rsh;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeCooperative;
  attr.val.cooperative = 1;  // every CTA resident at once: the barriers between the phases need it
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(m->token_grid);
  cfg.blockDim = dim3(kMoeThreads);
  cfg.dynamicSmemBytes = m->token_smem;
  cfg.stream = s;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  GOPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)m->token_smem));
  const cudaError_t e =
      cudaLaunchKernelEx(&cfg, kern, m->dev, rw ? reinterpret_cast<const uint4*>(rw->qweight) : (const uint4*)nullptr,
                         rw ? (const void*)rw->sb : (const void*)nullptr, rsh, rw ? m->hidden / rw->group_size : 0, x_dev,
                         logits_dev, m->logits, m->ids, m->wts, m->act, m->dpart, out_dev, m->bar, status, m->num_experts,
                         m->hidden, m->inter, m->top_k, m->norm_topk, sh, m->group_size);
  if (e == cudaErrorCooperativeLaunchTooLarge) {
    // the device cannot hold the grid at once (it is shared, or partitioned): this layer keeps to the
    // launches that need no co-residency from now on
    cudaGetLastError();
    m->token_grid = -1;
    *declined = true;
    return GOPH_OK;
  }
  if (e != cudaSuccess) return fail_cuda(e, "moe_token_kernel launch");
  note_launch();
  return GOPH_OK;
}

// Launches 2-5 for routing given as logits already on the device.
static int moe_entry_rows(const goph_moe_layer* m, int tokens) {
  // Tiled experts: items per work entry.  Two keep the narrow, faster form of the tensor-core kernel
  // (8 accumulator columns); from two items per expert on average entries of four, which read most
  // experts once, are faster (128 experts, top-8: 8 tokens 70.7 against 76.1 us, 32 tokens 133.8 against
  // 129.3 us).  Option moe_rows (2 or 4) overrides.
  int entry_rows = tokens * m->top_k < 2 * m->num_experts ? 2 : 4;
  if (options().moe_rows == 2 || options().moe_rows == 4) entry_rows = options().moe_rows;
  return entry_rows;
}

static MoeRouteArgs moe_route_args(goph_moe_layer* m, const float* logits_dev, int tokens) {
  MoeRouteArgs ra;
  memset(&ra, 0, sizeof ra);
  ra.logits = logits_dev;
  ra.num_experts = m->num_experts;
  ra.top_k = m->top_k;
  ra.norm_topk = m->norm_topk;
  ra.tokens = tokens;
  ra.max_tokens = m->max_tokens;
  ra.tb = m->dev;
  ra.ids = m->ids;
  ra.wts = m->wts;
  ra.lists = m->lists;
  ra.work = m->work;
  ra.items = m->items;
  ra.mwork = m->tiled == 1 ? m->mwork : nullptr;
  ra.max_entries = m->max_entries;
  ra.entry_rows = moe_entry_rows(m, tokens);
  return ra;
}

// routed: the routing kernel has already been launched (together with the router rows)
static int moe_run(goph_moe_layer* m, float* out_dev, const float* x_dev, const float* logits_dev, int tokens,
                   cudaStream_t s, bool routed = false) {
  if (int rc = moe_upload_tables(m)) return rc;
  const int sms = device_state(m->device).sm_count;
  const int entry_rows = moe_entry_rows(m, tokens);
  if (!routed) {
    if (int rc = moe_launch(moe_route_kernel, dim3(tokens), 128, 0, s, moe_route_args(m, logits_dev, tokens))) return rc;
  }
  if (m->tiled == 1) {
    // tiled experts: gate and up of every entry in one grouped launch of the tensor-core kernel, then
    // down (each launch preceded by the kernel that writes the entries' activations as digits)
    MmaGroupLaunch g;
    memset(&g, 0, sizeof g);
    g.work = m->mwork;
    g.count = m->lists + 2;
    g.entry_rows = entry_rows;
    g.max_entries = min(m->max_entries, min(tokens * m->top_k, m->num_experts * ((tokens + entry_rows - 1) / entry_rows)));
    g.top_k = m->top_k;
    g.xb = m->mxb;
    g.xtab = m->mxtab;
    g.first = 0;
    g.mats = 2;
    g.rows = m->inter;
    g.in_dim = m->hidden;
    g.phase = 0;
    g.src = x_dev;
    g.out = m->gu;
    if (int rc = mlx_mma_launch_grouped(m->device, g, s)) return rc;
    g.first = 2;
    g.mats = 1;
    g.rows = m->hidden;
    g.in_dim = m->inter;
    g.phase = 1;
    g.src = m->gu;
    g.out = m->dpart;
    if (int rc = mlx_mma_launch_grouped(m->device, g, s)) return rc;
    return moe_launch(moe_combine_kernel, dim3((m->hidden + 255) / 256, tokens), 256, 0, s, m->dev, m->dpart, m->ids, m->wts,
                      out_dev, m->hidden, m->top_k);
  }
  int sh = 0;
  while ((32 << sh) < m->group_size) ++sh;
  // at most this many experts can have been selected; CTAs past the actual number return at once
  const int max_active = min(m->num_experts, tokens * m->top_k);
  // two CTAs fit an SM.  One or two tokens: one wave, so the per-CTA staging of the vectors is paid
  // once; more tokens: two waves' worth of smaller CTAs even out experts with different item counts
  const int want_ctas = sms * (tokens <= 2 ? 2 : 4);
  for (int phase = 0; phase < 2; ++phase) {
    const int in_dim = phase == 0 ? m->hidden : m->inter, out_rows = phase == 0 ? m->inter : m->hidden;
    const int iters = (in_dim / 32 + 31) / 32;
    const size_t smem = (size_t)4 * iters * (256 * 16 + 32 * 8) + (size_t)kMoeWarps * kMoeDepth * kMoeStepBytes;
    if (smem > (size_t)kSmemBudget) return fail(GOPH_E_UNSUPPORTED, "MoE: %d columns do not fit shared memory", in_dim);
    const int tasks = phase == 0 ? out_rows : (out_rows + 1) / 2;
    const int max_blocks = (tasks + kMoeWarps - 1) / kMoeWarps;
    const int gx = max(1, min(max_blocks, (want_ctas + max_active - 1) / max_active));
    auto k = phase == 0 ? (m->sb_bf16 ? moe_expert_kernel<true, 0> : moe_expert_kernel<false, 0>)
                        : (m->sb_bf16 ? moe_expert_kernel<true, 1> : moe_expert_kernel<false, 1>);
    GOPH_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (int rc = moe_launch(k, dim3(gx, max_active), kMoeThreads, smem, s, m->work, m->lists, m->items,
                            phase == 0 ? x_dev : m->act, phase == 0 ? m->act : m->dpart, m->max_tokens, in_dim, out_rows,
                            m->top_k, sh, in_dim / m->group_size))
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
  const goph_mlx_weight* rw = m->router;
  MoeTokenKernel tk = nullptr;
  if (tokens == 1 && moe_token_form(m, rw, &tk)) {
    bool declined = false;
    const int rc = moe_run_token(m, tk, out_dev, x_dev, rw, nullptr, (cudaStream_t)stream, &declined);
    if (rc || !declined) return rc;
  }
  if (rw->qweight && rw->sb && rw->group_size >= 32 && !(rw->group_size & (rw->group_size - 1)) && rw->in_dim % 32 == 0) {
    // row-major router (the usual case: it is small): one launch for all tokens
    int sh = 0;
    while ((32 << sh) < rw->group_size) ++sh;
    const int iters = (m->hidden / 32 + 31) / 32;
    const size_t smem = (size_t)iters * (256 * 16 + 32 * 8);
    if (smem > (size_t)kSmemBudget) return fail(GOPH_E_UNSUPPORTED, "MoE: hidden=%d does not fit shared memory", m->hidden);
    const int cs = (m->num_experts + 2 * kMoeWarps - 1) / (2 * kMoeWarps);  // CTAs of a token: one per 16 experts
    if (cs <= 8 && options().moe_fused && !m->no_router_cluster) {
      // router rows and routing in one launch: the CTAs of a token form a thread-block cluster
      if (int rc = moe_upload_tables(m)) return rc;
      auto kr = rw->sb_bf16 ? moe_router_route_kernel<true> : moe_router_route_kernel<false>;
      GOPH_CUDA(cudaFuncSetAttribute(kr, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = options().pdl ? 1 : 0;
      attr[1].id = cudaLaunchAttributeClusterDimension;
      attr[1].val.clusterDim.x = cs;
      attr[1].val.clusterDim.y = 1;
      attr[1].val.clusterDim.z = 1;
      cudaLaunchConfig_t cfg;
      memset(&cfg, 0, sizeof cfg);
      cfg.gridDim = dim3(cs * tokens);
      cfg.blockDim = dim3(kMoeThreads);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = (cudaStream_t)stream;
      cfg.attrs = attr;
      cfg.numAttrs = cs > 1 ? 2 : 1;
      const cudaError_t e = cudaLaunchKernelEx(&cfg, kr, reinterpret_cast<const uint4*>(rw->qweight), (const void*)rw->sb, x_dev,
                                               m->logits, m->hidden, sh, m->hidden / rw->group_size, cs,
                                               moe_route_args(m, m->logits, tokens));
      if (e == cudaSuccess) {
        note_launch();
        return moe_run(m, out_dev, x_dev, m->logits, tokens, (cudaStream_t)stream, true);
      }
      // a device that does not take the cluster: the two launches below, for this layer from now on
      cudaGetLastError();
      m->no_router_cluster = 1;
    }
    auto k = rw->sb_bf16 ? moe_router_kernel<true> : moe_router_kernel<false>;
    GOPH_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (int rc = moe_launch(k, dim3((m->num_experts + 2 * kMoeWarps - 1) / (2 * kMoeWarps), tokens), kMoeThreads, smem,
                            (cudaStream_t)stream, reinterpret_cast<const uint4*>(rw->qweight), rw->sb, x_dev, m->logits,
                            m->num_experts, m->hidden, sh, m->hidden / rw->group_size))
      return rc;
  } else if (int rc = goph_mlx_gemm(m->logits, (uint64_t)tokens * m->num_experts, x_dev, x_len, rw, tokens, stream)) {
    return rc;
  }
  return moe_run(m, out_dev, x_dev, m->logits, tokens, (cudaStream_t)stream);
}

GOPH_API int goph_moe_forward_logits(goph_moe_layer* m, float* out_dev, uint64_t out_len, const float* x_dev,
                                     uint64_t x_len, const float* logits_dev, uint64_t logits_len, int tokens,
                                     void* stream) {
  clear_error();
  if (int rc = moe_check_io(m, out_dev, out_len, x_dev, x_len, tokens)) return rc;
  if (!logits_dev || logits_len < (uint64_t)tokens * m->num_experts) return fail(GOPH_E_INVALID, "router logits buffer too short");
  if (int rc = use_device(m->device)) return rc;
  MoeTokenKernel tk = nullptr;
  if (tokens == 1 && moe_token_form(m, nullptr, &tk)) {
    bool declined = false;
    const int rc = moe_run_token(m, tk, out_dev, x_dev, nullptr, logits_dev, (cudaStream_t)stream, &declined);
    if (rc || !declined) return rc;
  }
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

#ifdef GOPH_TUNING
GOPH_API int goph_tuning_probe_moe(long long* out16) {
  return cudaMemcpyFromSymbol(out16, g_moe_trace, 24 * sizeof(long long)) == cudaSuccess ? 0 : -1;
}
#endif
