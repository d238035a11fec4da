// FP8 E4M3FN linears with per-row (or per-tensor) f32 scales: upload, bit-exact
// dequantisation, and the dequant-fused GEMV / small-batch product.
//
// Replaces fp8_e4m3_gemv_f32 / fp8_e4m3_gemm_f32 / fp8_e4m3_dequant_transpose_f32 + sgemm_nn
// (backends/nvidia/ptx/fp8/fp8.go) behind nvidia.GemvFP8E4M3[Buffer] and
// GemmFP8E4M3[Buffer] (backends/nvidia/runtime/fp8.go:158-320, :995-1030).  Arithmetic
// specification: fp8.Linear.GemvTo (backends/simd/quant/fp8/fp8.go:219-239):
//     out[r] = (sum_j decode(W[r,j]) * x[j]) * scale[r] + bias[r].
// E4M3FN bytes are widened with the hardware converter (e4m3 → f16 → f32, both exact);
// the two NaN codes 0x7f / 0xff stay NaN, as in the reference's table (fp8.go:85-106).
#include <string.h>

#include "stream_gemv.cuh"
#include "tc_gemm.cuh"

namespace goph {

__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t two_bytes) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two_bytes & 0xFFFFu), __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

struct FP8Fmt {
  static constexpr int kSlots = 4;  // 16 elements per unit
  static constexpr bool kHasConsts = false;
  struct Row {
    uint4 q;
  };
  static __device__ __forceinline__ void load(const StreamArgs& a, int row, int unit, Row& t) {
    t.q = ld_stream(reinterpret_cast<const uint4*>(a.w + (size_t)row * a.in_dim) + unit);
  }
  static __device__ __forceinline__ float2 consts(float, float) { return make_float2(0.f, 0.f); }
  template <int M>
  static __device__ __forceinline__ void dot(const Row& t, const float4 (&xv)[M][4], const float2 (&)[M],
                                             float (&acc)[M]) {
    float2 F[M];
#pragma unroll
    for (int m = 0; m < M; ++m) F[m] = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t w = k == 0 ? t.q.x : k == 1 ? t.q.y : k == 2 ? t.q.z : t.q.w;
      float2 f0 = e4m3x2_to_float2(w), f1 = e4m3x2_to_float2(w >> 16);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float4 xa = xv[m][k];
        fma2(F[m], f0, make_float2(xa.x, xa.y));
        fma2(F[m], f1, make_float2(xa.z, xa.w));
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] += F[m].x + F[m].y;
  }
  static __device__ __forceinline__ float finish(const StreamArgs& a, int row, float v) {
    float o = __fmul_rn(v, reinterpret_cast<const float*>(a.aux)[row]);
    if (a.bias) o = __fadd_rn(o, a.bias[row]);
    return o;
  }
};


// Rows whose length is not a multiple of 16 bytes cannot be read as aligned 16-byte units:
// one warp per row, byte loads.
__global__ void __launch_bounds__(kGThreads)
fp8_gemv_ragged_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale,
                       const float* __restrict__ bias, const float* __restrict__ x, float* __restrict__ out,
                       int rows, int in_dim, int batch) {
  int row = blockIdx.x * kGWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  for (int m = 0; m < batch; ++m) {
    float acc = 0.f;
    for (int j = lane; j < in_dim; j += 32) {
      __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)w[(size_t)row * in_dim + j], __NV_E4M3);
      acc = fmaf(__half2float(*reinterpret_cast<__half*>(&h)), x[(size_t)m * in_dim + j], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      float o = __fmul_rn(acc, scale[row]);
      if (bias) o = __fadd_rn(o, bias[row]);
      out[(size_t)m * rows + row] = o;
    }
  }
}

// fp8.Linear.DequantRowTo: table value times the row scale, one rounding.
__global__ void fp8_dequant_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale,
                                   float* __restrict__ out, size_t n, int in_dim) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)w[i], __NV_E4M3);
  out[i] = __fmul_rn(__half2float(*reinterpret_cast<__half*>(&h)), scale[i / in_dim]);
}

__global__ void fp8_fill_scale_kernel(float* __restrict__ dst, const float* __restrict__ src, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[0];
}

static bool valid_fp8(const goph_fp8_linear* w) {
  return w && w->magic == kMagicFP8 && (w->weight || w->tiled) && w->scale && w->in_dim > 0 && w->out_dim > 0;
}

}  // namespace goph

using namespace goph;

GOPH_API int goph_fp8_upload(int device, const uint8_t* weight, uint64_t weight_len, const float* scale,
                             int scale_len, const float* bias, int bias_len, int out_dim, int in_dim,
                             goph_fp8_linear** out) {
  clear_error();
  if (!out) return fail(GOPH_E_INVALID, "goph_fp8_upload: nil result pointer");
  *out = nullptr;
  // fp8.Linear.Validate (backends/simd/quant/fp8/fp8.go:140-158).
  if (out_dim <= 0 || in_dim <= 0) return fail(GOPH_E_INVALID, "fp8 linear invalid dims out=%d in=%d", out_dim, in_dim);
  uint64_t want;
  if (!mul_ok((uint64_t)out_dim, (uint64_t)in_dim, &want))
    return fail(GOPH_E_INVALID, "fp8 linear weight size overflow out=%d in=%d", out_dim, in_dim);
  if (!weight || weight_len != want)
    return fail(GOPH_E_INVALID, "fp8 linear weight bytes=%llu want=%llu", (unsigned long long)weight_len,
                (unsigned long long)want);
  if (!scale || (scale_len != 1 && scale_len != out_dim))
    return fail(GOPH_E_INVALID, "fp8 linear scale len=%d want 1 or %d", scale_len, out_dim);
  if (bias && bias_len != out_dim) return fail(GOPH_E_INVALID, "fp8 linear bias len=%d want %d", bias_len, out_dim);
  if (int rc = use_device(device)) return rc;

  goph_fp8_linear* h = new goph_fp8_linear();
  memset(h, 0, sizeof *h);
  h->magic = kMagicFP8;
  h->device = device;
  h->in_dim = in_dim;
  h->out_dim = out_dim;
  h->scale_len = scale_len;
  float* tmp = nullptr;
  auto bail = [&](int rc) {
    cudaFree(tmp);
    if (rc) {
      cudaFree(h->weight);
      cudaFree(h->tiled);
      cudaFree(h->scale);
      cudaFree(h->bias);
      delete h;
    }
    return rc;
  };
#define UP(call)                                              \
  do {                                                        \
    cudaError_t _e = (call);                                  \
    if (_e != cudaSuccess) return bail(fail_cuda(_e, #call)); \
  } while (0)
  UP(cudaMalloc(&h->weight, want));
  UP(cudaMemcpy(h->weight, weight, want, cudaMemcpyHostToDevice));
  UP(cudaMalloc(&h->scale, (size_t)out_dim * 4));
  if (scale_len == 1) {
    UP(cudaMalloc(&tmp, 4));
    UP(cudaMemcpy(tmp, scale, 4, cudaMemcpyHostToDevice));
    fp8_fill_scale_kernel<<<(out_dim + 255) / 256, 256>>>(h->scale, tmp, out_dim);
    UP(cudaGetLastError());
  } else {
    UP(cudaMemcpy(h->scale, scale, (size_t)out_dim * 4, cudaMemcpyHostToDevice));
  }
  if (bias) {
    UP(cudaMalloc(&h->bias, (size_t)out_dim * 4));
    UP(cudaMemcpy(h->bias, bias, (size_t)out_dim * 4, cudaMemcpyHostToDevice));
  }
  UP(cudaDeviceSynchronize());
#undef UP
  h->bytes = want + (uint64_t)out_dim * 4 * (bias ? 2 : 1);
  // Tensor-core layout for matrices large enough to amortise that path's fixed cost; a matrix
  // holding one of the two NaN codes stays row-major (the kernel that serves large bf16 batches
  // turns the bytes into bf16 and would map those codes to +-480; the CUDA-core kernels keep them
  // NaN as the reference's table does).
  const bool big = want >= (8u << 20);
  if (tc_fp8_supported(in_dim) && (options().fp8_layout == 2 || (options().fp8_layout == 0 && big))) {
    int has_nan = 0;
    if (int rc = tc_fp8_make_tiled(h, &has_nan)) return bail(rc);
    if (h->tiled) {
      cudaFree(h->weight);
      h->weight = nullptr;
      h->bytes = (uint64_t)((out_dim + 127) / 128) * 128 * in_dim + (uint64_t)out_dim * 4 * (bias ? 2 : 1);
    }
  }
  *out = h;
  return bail(GOPH_OK);
}

GOPH_API int goph_fp8_free(goph_fp8_linear* w) {
  clear_error();
  if (!w) return GOPH_OK;
  if (w->magic != kMagicFP8) return fail(GOPH_E_INVALID, "goph_fp8_free: not an FP8 linear handle");
  if (int rc = use_device(w->device)) return rc;
  cudaFree(w->weight);
  cudaFree(w->tiled);
  cudaFree(w->scale);
  cudaFree(w->bias);
  w->magic = 0;
  delete w;
  return GOPH_OK;
}

GOPH_API uint64_t goph_fp8_resident_bytes(const goph_fp8_linear* w) {
  return (w && w->magic == kMagicFP8) ? w->bytes : 0;
}

GOPH_API int goph_fp8_dequant(const goph_fp8_linear* w, float* out_dev, uint64_t out_len, void* stream) {
  clear_error();
  if (!valid_fp8(w)) return fail(GOPH_E_INVALID, "invalid FP8 linear handle");
  uint64_t need = (uint64_t)w->out_dim * w->in_dim;
  if (!out_dev || out_len < need)
    return fail(GOPH_E_INVALID, "dequant out length=%llu, want at least %llu", (unsigned long long)out_len,
                (unsigned long long)need);
  if (int rc = use_device(w->device)) return rc;
  if (w->tiled) return tc_fp8_dequant_tiled(w, out_dev, (cudaStream_t)stream);
  fp8_dequant_kernel<<<(unsigned)((need + 255) / 256), 256, 0, (cudaStream_t)stream>>>(w->weight, w->scale, out_dev,
                                                                                       need, w->in_dim);
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

GOPH_API int goph_fp8_gemm(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len, int batch,
                           const goph_fp8_linear* w, void* stream) {
  clear_error();
  if (!valid_fp8(w)) return fail(GOPH_E_INVALID, "invalid FP8 linear handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_x, need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)w->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)w->out_dim, &need_o))
    return fail(GOPH_E_INVALID, "fp8 batch size overflow batch=%d in=%d out=%d", batch, w->in_dim, w->out_dim);
  if (!x_dev || x_len < need_x || !out_dev || out_len < need_o)
    return fail(GOPH_E_INVALID, "fp8 batch buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len,
                (unsigned long long)need_x, (unsigned long long)out_len, (unsigned long long)need_o);
  if (int rc = use_device(w->device)) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  // Tensor-core layout: every batch size goes to the kernel that feeds the e4m3 bytes to the MMA as
  // they lie (fp8_mma.cu); the row-major layout is served by the CUDA-core kernels below.
  if (w->tiled) return tc_gemm_fp8(w, out_dev, x_dev, false, batch, s);
  if (!w->tiled && w->in_dim % 16 != 0) {
    note_launch();
    fp8_gemv_ragged_kernel<<<(w->out_dim + kGWarps - 1) / kGWarps, kGThreads, 0, s>>>(
        w->weight, w->scale, w->bias, x_dev, out_dev, w->out_dim, w->in_dim, batch);
    GOPH_CUDA(cudaGetLastError());
    return GOPH_OK;
  }
  StreamArgs a;
  memset(&a, 0, sizeof a);
  a.w = w->weight;
  a.aux = w->scale;
  a.bias = w->bias;
  a.out = out_dev;
  a.x = x_dev;
  a.rows = w->out_dim;
  a.in_dim = w->in_dim;
  a.units = w->in_dim / 16;
  a.row_bytes = w->in_dim;
  const int force_rows = options().fp8_rows;
  return stream_launch<FP8Fmt>(a, w->device, batch, s, force_rows);
}

GOPH_API int goph_fp8_gemm_bf16(float* out_dev, uint64_t out_len, const uint16_t* x_bf16_dev, uint64_t x_len, int batch,
                                const goph_fp8_linear* w, void* stream) {
  clear_error();
  if (!valid_fp8(w)) return fail(GOPH_E_INVALID, "invalid FP8 linear handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_x, need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)w->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)w->out_dim, &need_o))
    return fail(GOPH_E_INVALID, "fp8 batch size overflow batch=%d in=%d out=%d", batch, w->in_dim, w->out_dim);
  if (!x_bf16_dev || x_len < need_x || !out_dev || out_len < need_o)
    return fail(GOPH_E_INVALID, "fp8 batch buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len,
                (unsigned long long)need_x, (unsigned long long)out_len, (unsigned long long)need_o);
  if (!w->tiled)
    return fail(GOPH_E_UNSUPPORTED,
                "goph_fp8_gemm_bf16 needs a linear in the tensor-core layout (in_dim a multiple of 256, no NaN codes, "
                "uploaded with fp8_layout 0 or 2)");
  if (int rc = use_device(w->device)) return rc;
  return tc_gemm_fp8(w, out_dev, x_bf16_dev, true, batch, (cudaStream_t)stream);
}

GOPH_API int goph_fp8_gemm_host(float* out_host, uint64_t out_len, const float* x_host, uint64_t x_len, int batch,
                                const goph_fp8_linear* w) {
  clear_error();
  if (!valid_fp8(w)) return fail(GOPH_E_INVALID, "invalid FP8 linear handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_x, need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)w->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)w->out_dim, &need_o))
    return fail(GOPH_E_INVALID, "fp8 batch size overflow");
  if (!x_host || x_len < need_x || !out_host || out_len < need_o)
    return fail(GOPH_E_INVALID, "fp8 batch buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len,
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
  if (!rc) rc = goph_fp8_gemm(dout, need_o, dx, need_x, batch, w, nullptr);
  if (!rc) {
    e = cudaMemcpy(out_host, dout, need_o * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) rc = fail_cuda(e, "cudaMemcpy(out)");
  }
  cudaFree(dx);
  cudaFree(dout);
  return rc;
}
