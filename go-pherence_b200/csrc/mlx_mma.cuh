// Tensor-core (tcgen05) path for MLX 4-bit weights; implemented in mlx_mma.cu.
#pragma once

#include "goph_internal.cuh"

namespace goph {

// True when the weight's layout meets the tensor-map constraints of the tensor-core kernel
// (bf16 scale/bias table, group size 64, in_dim a multiple of 256, 16-byte aligned buffers).
bool mlx_mma_supported(const goph_mlx_weight* w);
// Encodes the two TMA tensor maps of a weight (packed nibbles, {scale,bias} pairs).
int mlx_mma_make_maps(goph_mlx_weight* w);
void mlx_mma_free_maps(goph_mlx_weight* w);
// out[batch][out_dim] = x[batch][in_dim] * W^T.  pieces: bf16 pieces per activation (3 = any
// f32 exactly, 1 = x already holds bf16 values).
int mlx_mma_launch(const goph_mlx_weight* w, float* out, const float* x, int batch, int pieces, cudaStream_t stream);
// Reads the device status word (0 = every wait completed); synchronises the copy stream.
int mlx_mma_status(int device);

}  // namespace goph
