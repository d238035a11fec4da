// Tensor-core (tcgen05) path for MLX 4-bit weights; implemented in mlx_mma.cu.
#pragma once

#include "goph_internal.cuh"

namespace goph {

// True when the weight's shape allows the tiled layout of the tensor-core kernel (bf16
// scale/bias table, group size 64, in_dim a multiple of 256).
bool mlx_mma_supported(const goph_mlx_weight* w);
// Builds the tiled copy from the row-major buffers of w (which the caller then frees).
int mlx_mma_make_tiled(goph_mlx_weight* w);
// Byte offsets inside the tiled layout (shared with the dequantisation kernel).
constexpr int kMlxTileRows = 128, kMlxChunkK = 256, kMlxBlockW = 128 * 128, kMlxBlockBytes = 128 * 128 + 128 * 16;
__host__ __device__ inline size_t mlx_tiled_word_offset(int row, int col, int nchunks) {
  size_t blk = (size_t)(row >> 7) * nchunks + (col >> 8);
  int r = row & 127, u = (col & 255) >> 5, w = (col & 31) >> 3;
  return blk * kMlxBlockBytes + r * 128 + ((u ^ (r & 7)) << 4) + w * 4;
}
__host__ __device__ inline size_t mlx_tiled_meta_offset(int row, int col, int nchunks) {
  size_t blk = (size_t)(row >> 7) * nchunks + (col >> 8);
  return blk * kMlxBlockBytes + kMlxBlockW + (row & 127) * 16 + ((col & 255) >> 6) * 4;
}
// out[batch][out_dim] = x[batch][in_dim] * W^T.  digits: base-128 digits each activation is
// written in (4 = 27 bits under the group maximum, 3 = 20 bits).  x_prepared: the previous
// launch on this stream prepared the same x (same batch, same in_dim), skip the preparation.
int mlx_mma_launch(const goph_mlx_weight* w, float* out, const float* x, int batch, int digits, cudaStream_t stream,
                   bool x_prepared = false);

// ---- grouped launches: the selected experts of a mixture-of-experts layer --------------------
// One work entry = one expert (tiled matrices of equal shapes) and up to `rows` (2 or 4, the same
// for every entry of a call) of the (token, slot) items that chose it; an expert chosen by more
// items has several entries.
constexpr int kMoeMmaRowsMin = 2, kMoeMmaRowsMax = 4;
struct __align__(16) MmaGroupEntry {
  const unsigned char* w[3];  // tiled gate, up, down
  int count;                  // items of this entry, 1..rows
  int expert;
  int item[8];                // token * top_k + slot
};
// True when experts of [inter x hidden] / [hidden x inter] can run as grouped launches.
bool mlx_mma_grouped_supported(int hidden, int inter);
// Bytes of prepared activations and floats of tables one entry of `rows` items needs for an input of in_dim.
size_t mlx_mma_grouped_xb_bytes(int in_dim, int rows);
int mlx_mma_grouped_tab_floats(int in_dim, int rows);
struct MmaGroupLaunch {
  const MmaGroupEntry* work;  // device
  const int* count;           // device: live entries
  int max_entries;            // entries the launch is sized for
  int entry_rows;             // items per entry: 2 or 4
  int first, mats;            // matrices of an entry this launch multiplies: w[first .. first + mats)
  int rows, in_dim;           // shape of each of them
  int phase;                  // 0: activations = row item / top_k of src; 1: silu(g) * u of src's row entry * entry_rows + m
  int top_k;
  const float* src;
  unsigned char* xb;          // [max_entries][xb_bytes]
  float* xtab;                // [max_entries][tab_floats]
  float* out;                 // phase 0: [max_entries * entry_rows][mats * rows]; phase 1: [items][rows]
};
// Two launches: the entries' activations as digits, sums and scales; then the products.
int mlx_mma_launch_grouped(int device, const MmaGroupLaunch& g, cudaStream_t stream);

// Reads the device status word (0 = every wait completed); synchronises the copy stream.
int mlx_mma_status(int device);
void mlx_mma_status_clear(int device);

// GGUF Q4_K / Q8_0 on the same kernel.  make_tiled builds m->tiled from the matrix's device
// buffers (which the caller then frees); dequant reproduces dequantRowQ4KTo / dequantRowQ8_0To.
bool gguf_mma_supported(int qtype, int in_dim);
int gguf_mma_make_tiled(goph_gguf_matrix* m);
// x_prepared: the launch in front on this stream prepared the same x for a matrix of the same type
// (same batch, same in_dim): the preparation kernel is skipped.
int gguf_mma_launch(const goph_gguf_matrix* m, float* out, const float* x, int batch, int digits, cudaStream_t stream,
                    bool x_prepared = false);
int gguf_mma_dequant(const goph_gguf_matrix* m, float* out, cudaStream_t stream);

}  // namespace goph
