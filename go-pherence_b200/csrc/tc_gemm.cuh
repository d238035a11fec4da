// Small-batch products (prefill chunks, verifier batches: 9..256 activation rows) on the tensor
// cores with bf16 operands and f32 accumulation; implemented in tc_gemm.cu.
#pragma once

#include "goph_internal.cuh"

namespace goph {

// MLX 4-bit weight in the tiled layout (see goph_mlx_weight).  x is [batch][in_dim], either f32
// (x_bf16 = false: every element is split into three bf16 pieces, exact) or bf16 bit patterns
// (x_bf16 = true: one piece).  out is [batch][out_dim] f32.
int tc_gemm_mlx(const goph_mlx_weight* w, float* out, const void* x, bool x_bf16, int batch, cudaStream_t stream);

// FP8 E4M3 linear in the tensor-core layout (goph_fp8_linear::tiled), any batch size; implemented
// in fp8_mma.cu (e4m3 operands read by the MMA from shared memory, nothing converted).
int tc_gemm_fp8(const goph_fp8_linear* w, float* out, const void* x, bool x_bf16, int batch, cudaStream_t stream);

// The same product through the bf16 kernel of tc_gemm.cu (the e4m3 bytes are turned into bf16 on the
// way to the tensor cores): the faster of the two for bf16 activations of more than 32 rows.
int tc_gemm_fp8_converted(const goph_fp8_linear* w, float* out, const void* x, bool x_bf16, int batch, cudaStream_t stream);

// True when an FP8 linear of this shape can take the tiled layout (in_dim a multiple of 256).
bool tc_fp8_supported(int in_dim);
// Builds w->tiled from w->weight (row-major bytes on the device); the caller then frees w->weight.
// Sets *has_nan when a byte is one of the two NaN codes (such a matrix stays row-major).
int tc_fp8_make_tiled(goph_fp8_linear* w, int* has_nan);
// fp8.Linear.DequantRowTo from the tiled layout.
int tc_fp8_dequant_tiled(const goph_fp8_linear* w, float* out, cudaStream_t stream);
// K splits per 128-row tile for a persistent grid of `sms` CTAs (see tc_gemm.cu).
int tc_choose_splits(int ntiles, int nchunks, int sms, int max_items, float fix_cost);
// Device status word of the small-batch kernels (0 = every wait completed).
int tc_gemm_status(int device);
void tc_gemm_status_clear(int device);
// The same for the FP8 kernel of fp8_mma.cu.
int fp8_mma_status(int device);
void fp8_mma_status_clear(int device);

}  // namespace goph
