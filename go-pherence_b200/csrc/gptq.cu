// GPTQ symmetric INT4 weights (nvidia.GPUQuantWeight, backends/nvidia/runtime/q4.go:18-26;
// arithmetic of backends/simd/quant/q4/gemv.go:76-94): weight[j][i] = scales[g_idx[i]][j] * (q - 8)
// with q the nibble of input i in qweight[i/8][j].
//
// The checkpoint layout ([in/8][out] words, [groups][out] scales) is turned at upload into rows:
// words [out][in/8] (the nibble order inside a word is already the one the MLX kernels read) and
// scales [out][groups].  Two cases:
//   regular g_idx (g_idx[i] == i / gs for equal groups of gs inputs, gs a multiple of 8): q*s - 8*s is the MLX affine
//     form with bias = -8*s, which is exact in f32, so the weight becomes an MLX weight handle and
//     every MLX kernel (tensor-core path included) serves it;
//   any other g_idx (act-order checkpoints, unequal groups): a warp-per-row kernel that looks the
//     scale up per input through g_idx.
#include <vector>

#include "goph_internal.cuh"

using namespace goph;

constexpr uint32_t kMagicGPTQ = 0x47505451;  // "GPTQ"

struct goph_gptq_weight {
  uint32_t magic;
  int device;
  int in_dim, out_dim, groups;
  goph_mlx_weight* mlx;  // regular g_idx: the whole weight lives here
  int exact_affine;      // q*s + (-8*s) equals s*(q-8) for every scale (low four mantissa bits clear)
  uint32_t* words;       // [out][in/8]           (irregular g_idx only)
  float* scales;         // [out][groups]         (irregular g_idx, or regular with exact_affine == 0)
  int* gidx;             // [in]                  (irregular g_idx only)
  uint64_t bytes;
};

namespace {

constexpr int kWarps = 8;

// One warp per output row; lanes stride over the row's packed words.  Scales are fetched per input
// through g_idx (L1-resident: a row's scales are contiguous).
template <int M>
__global__ void __launch_bounds__(kWarps * 32)
gptq_rows_kernel(const uint32_t* __restrict__ words, const float* __restrict__ scales, const int* __restrict__ gidx,
                 const float* __restrict__ x, float* __restrict__ out, int in_dim, int out_dim, int groups) {
  const int row = blockIdx.x * kWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= out_dim) return;
  const uint32_t* wr = words + (size_t)row * (in_dim / 8);
  const float* sr = scales + (size_t)row * groups;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  for (int p = lane; p < in_dim / 8; p += 32) {
    const uint32_t w = __ldg(wr + p);
    const int4 g0 = __ldg(reinterpret_cast<const int4*>(gidx + 8 * p));
    const int4 g1 = __ldg(reinterpret_cast<const int4*>(gidx + 8 * p + 4));
    const int g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    float wv[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) wv[k] = __ldg(sr + g[k]) * (float)((int)((w >> (4 * k)) & 0xFu) - 8);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float4 xa = __ldg(reinterpret_cast<const float4*>(x + (size_t)m * in_dim + 8 * p));
      const float4 xb = __ldg(reinterpret_cast<const float4*>(x + (size_t)m * in_dim + 8 * p + 4));
      float s = acc[m];
      s = fmaf(xa.x, wv[0], s); s = fmaf(xa.y, wv[1], s); s = fmaf(xa.z, wv[2], s); s = fmaf(xa.w, wv[3], s);
      s = fmaf(xb.x, wv[4], s); s = fmaf(xb.y, wv[5], s); s = fmaf(xb.z, wv[6], s); s = fmaf(xb.w, wv[7], s);
      acc[m] = s;
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float v = acc[m];
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) out[(size_t)m * out_dim + row] = v;
  }
}

// q4.DequantSymTo: out[j*in + i] = scale * float32(q - 8), one rounding.
__global__ void gptq_dequant_kernel(const uint32_t* __restrict__ words, const float* __restrict__ scales,
                                    const int* __restrict__ gidx, float* __restrict__ out, int in_dim, int out_dim,
                                    int groups, int gs) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)out_dim * (in_dim / 8)) return;
  const size_t row = idx / (in_dim / 8), p = idx - row * (in_dim / 8);
  const uint32_t w = words[idx];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = (int)p * 8 + k;
    const int g = gidx ? gidx[i] : i / gs;
    out[row * in_dim + i] = __fmul_rn(scales[row * groups + g], (float)((int)((w >> (4 * k)) & 0xFu) - 8));
  }
}

bool valid_gptq(const goph_gptq_weight* w) {
  return w && w->magic == kMagicGPTQ && w->in_dim > 0 && w->out_dim > 0 && w->groups > 0 && (w->mlx || (w->words && w->scales && w->gidx));
}

void release(goph_gptq_weight* w) {
  if (w->mlx) goph_mlx_free(w->mlx);
  cudaFree(w->words);
  cudaFree(w->scales);
  cudaFree(w->gidx);
  w->mlx = nullptr;
  w->words = nullptr;
  w->scales = nullptr;
  w->gidx = nullptr;
  w->magic = 0;
  delete w;
}

template <int M>
void launch_rows(const goph_gptq_weight* w, const float* x, float* out, cudaStream_t s) {
  note_launch();
  gptq_rows_kernel<M><<<(w->out_dim + kWarps - 1) / kWarps, kWarps * 32, 0, s>>>(w->words, w->scales, w->gidx, x, out,
                                                                               w->in_dim, w->out_dim, w->groups);
}

}  // namespace

GOPH_API int goph_gptq_upload(int device, const int32_t* qweight, uint64_t qweight_len, const int32_t* g_idx,
                              uint64_t g_idx_len, const float* scales, uint64_t scales_len, int in_dim, int out_dim,
                              goph_gptq_weight** out) {
  clear_error();
  if (!out) return fail(GOPH_E_INVALID, "goph_gptq_upload: nil result pointer");
  *out = nullptr;
  if (in_dim <= 0 || out_dim <= 0 || in_dim % 8 != 0)
    return fail(GOPH_E_INVALID, "invalid Q4 dims inDim=%d outDim=%d", in_dim, out_dim);
  uint64_t want_q;
  if (!mul_ok((uint64_t)(in_dim / 8), (uint64_t)out_dim, &want_q) || want_q > (UINT64_MAX >> 3))
    return fail(GOPH_E_INVALID, "qweight size overflow for inDim=%d outDim=%d", in_dim, out_dim);
  if (!qweight || qweight_len < want_q)
    return fail(GOPH_E_INVALID, "qweight length=%llu, want at least %llu", (unsigned long long)qweight_len,
                (unsigned long long)want_q);
  if (!g_idx || g_idx_len < (uint64_t)in_dim)
    return fail(GOPH_E_INVALID, "gIdx length=%llu, want at least %d", (unsigned long long)g_idx_len, in_dim);
  if (!scales || scales_len == 0 || scales_len % (uint64_t)out_dim != 0)
    return fail(GOPH_E_INVALID, "scales length=%llu is not a positive multiple of outDim=%d",
                (unsigned long long)scales_len, out_dim);
  const uint64_t groups64 = scales_len / (uint64_t)out_dim;
  if (groups64 > (uint64_t)INT32_MAX) return fail(GOPH_E_INVALID, "scales size overflow groups=%llu outDim=%d",
                                                  (unsigned long long)groups64, out_dim);
  const int groups = (int)groups64;
  for (int i = 0; i < in_dim; ++i)
    if (g_idx[i] < 0 || g_idx[i] >= groups)
      return fail(GOPH_E_INVALID, "gIdx[%d]=%d out of range [0,%d)", i, g_idx[i], groups);
  if (int rc = use_device(device)) return rc;

  bool regular = in_dim % groups == 0 && (in_dim / groups) % 8 == 0;
  const int gs = regular ? in_dim / groups : 0;
  for (int i = 0; regular && i < in_dim; ++i) regular = g_idx[i] == i / gs;

  // rows: words [out][in/8], scales [out][groups]
  const int packs = in_dim / 8;
  std::vector<uint32_t> words((size_t)out_dim * packs);
  std::vector<float> st((size_t)out_dim * groups);
  for (int p = 0; p < packs; ++p)
    for (int j = 0; j < out_dim; ++j) words[(size_t)j * packs + p] = (uint32_t)qweight[(size_t)p * out_dim + j];
  bool exact = true;
  for (int g = 0; g < groups; ++g)
    for (int j = 0; j < out_dim; ++j) {
      const float s = scales[(size_t)g * out_dim + j];
      uint32_t bits;
      memcpy(&bits, &s, 4);
      // q*s needs four more mantissa bits than s; with the low four clear (and s not subnormal) it is exact
      if ((bits & 0xFu) != 0 || ((bits >> 23) & 0xFFu) == 0) exact = exact && s == 0.f;
      st[(size_t)j * groups + g] = s;
    }

  auto* h = new goph_gptq_weight();
  h->magic = kMagicGPTQ;
  h->device = device;
  h->in_dim = in_dim;
  h->out_dim = out_dim;
  h->groups = groups;
  h->exact_affine = exact ? 1 : 0;
  auto bail = [&](int rc) {
    release(h);
    return rc;
  };
  auto put = [&](void** dst, const void* src, size_t bytes) -> int {
    cudaError_t e = cudaMalloc(dst, bytes);
    if (e != cudaSuccess) return fail_cuda(e, "cudaMalloc(gptq)");
    e = cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpy(gptq)");
    h->bytes += bytes;
    return GOPH_OK;
  };
  if (regular) {
    std::vector<float> bias(st.size());
    for (size_t k = 0; k < st.size(); ++k) bias[k] = -8.f * st[k];
    if (int rc = goph_mlx_upload(device, words.data(), words.size(), st.data(), bias.data(), st.size(), in_dim, out_dim,
                                 gs, &h->mlx))
      return bail(rc);
    h->bytes = goph_mlx_resident_bytes(h->mlx);
    if (!exact) {  // the bit-exact dequantisation then needs the f32 scales and the row-major words
      if (int rc = put((void**)&h->scales, st.data(), st.size() * 4)) return bail(rc);
      if (int rc = put((void**)&h->words, words.data(), words.size() * 4)) return bail(rc);
    }
  } else {
    if (int rc = put((void**)&h->words, words.data(), words.size() * 4)) return bail(rc);
    if (int rc = put((void**)&h->scales, st.data(), st.size() * 4)) return bail(rc);
    if (int rc = put((void**)&h->gidx, g_idx, (size_t)in_dim * 4)) return bail(rc);
  }
  *out = h;
  return GOPH_OK;
}

GOPH_API int goph_gptq_free(goph_gptq_weight* w) {
  clear_error();
  if (!w) return GOPH_OK;
  if (w->magic != kMagicGPTQ) return fail(GOPH_E_INVALID, "goph_gptq_free: not a GPTQ weight handle");
  if (int rc = use_device(w->device)) return rc;
  release(w);
  return GOPH_OK;
}

GOPH_API uint64_t goph_gptq_resident_bytes(const goph_gptq_weight* w) { return valid_gptq(w) ? w->bytes : 0; }

GOPH_API int goph_gptq_uses_mlx_kernels(const goph_gptq_weight* w) { return valid_gptq(w) && w->mlx ? 1 : 0; }

GOPH_API int goph_gptq_gemm(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len, int batch,
                            const goph_gptq_weight* w, void* stream) {
  clear_error();
  if (!valid_gptq(w)) return fail(GOPH_E_INVALID, "invalid Q4 weight handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_x, need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)w->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)w->out_dim, &need_o))
    return fail(GOPH_E_INVALID, "Q4 batch size overflow batch=%d in=%d out=%d", batch, w->in_dim, w->out_dim);
  if (!x_dev || x_len < need_x || !out_dev || out_len < need_o)
    return fail(GOPH_E_INVALID, "Q4 batch buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len,
                (unsigned long long)need_x, (unsigned long long)out_len, (unsigned long long)need_o);
  if (w->mlx) return goph_mlx_gemm(out_dev, out_len, x_dev, x_len, w->mlx, batch, stream);
  if (int rc = use_device(w->device)) return rc;
  if ((uintptr_t)x_dev % 16) return fail(GOPH_E_INVALID, "Q4 activations must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  for (int b = 0; b < batch;) {
    const int m = batch - b >= 4 ? 4 : batch - b >= 2 ? 2 : 1;
    const float* x = x_dev + (size_t)b * w->in_dim;
    float* o = out_dev + (size_t)b * w->out_dim;
    if (m == 4) launch_rows<4>(w, x, o, s);
    else if (m == 2) launch_rows<2>(w, x, o, s);
    else launch_rows<1>(w, x, o, s);
    b += m;
  }
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

GOPH_API int goph_gptq_dequant(const goph_gptq_weight* w, float* out_dev, uint64_t out_len, void* stream) {
  clear_error();
  if (!valid_gptq(w)) return fail(GOPH_E_INVALID, "invalid Q4 weight handle");
  uint64_t need;
  if (!mul_ok((uint64_t)w->in_dim, (uint64_t)w->out_dim, &need) || !out_dev || out_len < need)
    return fail(GOPH_E_INVALID, "dequant out length=%llu, want at least %llu", (unsigned long long)out_len,
                (unsigned long long)(uint64_t)w->in_dim * w->out_dim);
  if (w->mlx && w->exact_affine) return goph_mlx_dequant(w->mlx, out_dev, out_len, stream);
  if (int rc = use_device(w->device)) return rc;
  const size_t n = (size_t)w->out_dim * (w->in_dim / 8);
  gptq_dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      w->words, w->scales, w->gidx, out_dev, w->in_dim, w->out_dim, w->groups, w->mlx ? w->in_dim / w->groups : 1);
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}
