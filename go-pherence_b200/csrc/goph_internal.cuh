// Internal declarations shared by the translation units of libgoph_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/goph_b200.h"

#define GOPH_API extern "C" __attribute__((visibility("default")))

namespace goph {

constexpr int kMaxDevices = 16;
constexpr uint32_t kMagicMLX = 0x4d4c5834;   // "MLX4"
constexpr uint32_t kMagicGGUF = 0x47475546;  // "GGUF"
constexpr uint32_t kMagicFP8 = 0x46503845;   // "FP8E"

struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int max_smem_optin = 0;  // bytes of dynamic shared memory a CTA may opt into
};

DeviceState& device_state(int device);

// Error plumbing: every failure records a message for goph_last_error().
int fail(int code, const char* fmt, ...);
int fail_cuda(cudaError_t e, const char* what);
void clear_error();

#define GOPH_CUDA(call)                                   \
  do {                                                    \
    cudaError_t _e = (call);                              \
    if (_e != cudaSuccess) return goph::fail_cuda(_e, #call); \
  } while (0)

// Binds `device` for the calling thread and checks goph_init was done.
int use_device(int device);

// Overflow-checked product (internal/checked.MulInt in the reference).
inline bool mul_ok(uint64_t a, uint64_t b, uint64_t* out) {
  if (a != 0 && b > UINT64_MAX / a) return false;
  *out = a * b;
  return true;
}

// Tuning switches set through goph_set_option.
struct Options {
  int pdl = 1;         // launch kernels with programmatic stream serialization
  int mlx_layout = 0;  // layout chosen at upload: 0 by size, 1 always row-major, 2 tiled whenever the shape allows
  int mlx_splits = 0;  // K splits on the tensor-core path (0 = by shape)
  int mlx_fuse = 1;    // 1: narrow tensor-core launches make the activation digits of their own K range themselves (one launch)
  int mlx_chunks = 0;  // 1: one 256-element chunk per pipeline stage of the tensor-core GEMV; 0: two where the format allows
  int moe_fused = 1;   // MoE call of one token with row-major experts: 1 one cooperative launch, 0 the five launches of any token count
  int moe_rows = 0;    // tiled MoE experts: items per work entry (2 or 4); 0 = by the number of tokens
  int mlx_cluster = 1; // 1: K splits that run in one wave exchange their partial sums inside a thread-block cluster; 0: always through global scratch
  int mlx_digits = 4;  // base-128 digits per activation on the tensor-core path (4: 27 bits, 3: 20 bits)
  int mlx_unpack = 0;
  int gguf_layout = 0; // as mlx_layout, for Q4_K / Q8_0 matrices
  int fp8_layout = 0;  // as mlx_layout, for FP8 linears
  int fp8_convert = 0; // 1: bf16 batches above 32 rows of a tensor-core FP8 linear go through the kernel that turns e4m3 into bf16
  int mlx_rows = 0, gguf_rows = 0, fp8_rows = 0;
  int mlx_ctas_per_sm = 0;  // tuning aid: cap on resident CTAs per SM of the MLX streaming kernel and of product lists (0 = by shape)
};
Options& options();

// Counts a compute-kernel launch made for the caller (goph_launch_count reads the total).
void note_launch();

// Status word of the decode-step kernels on the current device (0, or 401 / 402 when a kernel found
// the position word outside [0, max_seq)).
int decode_ops_status();
void decode_ops_status_clear();

// Status word of the work-list kernels of gguf_work.cu (0, 601: an expert index outside the matrix,
// 602: a destination outside dst).
int gguf_work_status(int device);
int moe_status(int device);
void moe_status_clear(int device);
void gguf_work_status_clear(int device);

// Largest dynamic shared-memory request the GEMV kernels make.
constexpr int kSmemBudget = 200 * 1024;

}  // namespace goph

// MLX weight resident on one GPU, in one of two layouts:
//  row-major  packed words in the checkpoint's own order [out][in/8] (qweight) plus a table of
//             {scale,bias} pairs [out][groups] (sb) — the CUDA-core kernels' layout;
//  tiled      (tiled != nullptr; qweight and sb are then null) one 18 KiB block per 128 rows x
//             256 elements, blocks ordered [tile][chunk]: 128 rows x 128 packed bytes stored as the
//             shared-memory image the tensor-core kernel wants (16-byte unit u of row r at
//             r*128 + ((u ^ (r & 7)) << 4)), then 128 x 16 bytes of bf16 {scale,bias} pairs.  Rows
//             past out_dim are zero.  One stage of the kernel is one contiguous block.
struct goph_mlx_weight {
  uint32_t magic;
  int device;
  int in_dim, out_dim, group_size, groups;
  int sb_bf16;          // 1: sb is __nv_bfloat162 {scale,bias}; 0: float2 {scale,bias}
  uint32_t* qweight;    // [out_dim][in_dim/8]
  void* sb;             // [out_dim][groups]
  uint8_t* tiled;       // tiled layout or nullptr
  uint64_t bytes;
};

// GGUF matrix resident on one GPU, re-laid out at upload (same byte count as the file):
//  Q4_K: 144-byte super-blocks; 16-byte header {f16 d, f16 dmin, 8 x 12-bit (sc | m<<6)}
//        followed by 8 x 16 bytes, sub-block s in bytes [16s,16s+16), element 2i of the
//        sub-block in the low nibble of byte i and element 2i+1 in the high nibble.
//  Q8_0: int8 plane [out][in] stored with +128 bias (unsigned), then f16 d [out][in/32].
struct goph_gguf_matrix {
  uint32_t magic;
  int device;
  int qtype, in_dim, out_dim;
  uint8_t* data;   // Q4_K, Q5_K: blocks; Q8_0: biased int8 plane; Q6_K: low-nibble plane
  uint16_t* d16;   // Q8_0: f16 scales; Q6_K: two-bit highs, int8 scales and f16 d, one plane after another
  uint8_t* tiled;  // tensor-core layout (data and d16 are then null): one stage per 128 rows x 256 elements
  uint64_t bytes;
};

// FP8 E4M3 linear resident on one GPU: bytes as uploaded, per-row f32 scale (a per-tensor
// scale is broadcast at upload), optional f32 bias.
struct goph_fp8_linear {
  uint32_t magic;
  int device;
  int in_dim, out_dim;
  int scale_len;      // what the caller passed (1 or out_dim)
  uint8_t* weight;    // [out_dim][in_dim] (row-major layout) or nullptr
  uint8_t* tiled;     // tensor-core layout or nullptr: one 32 KiB block per 128 rows x 256 bytes, blocks
                      // ordered [tile][chunk], 16-byte unit u of row r at (u/2)*4096 + (u%2)*2048 + (r/8)*128 + (r%8)*16
                      // (the K-major 8 x 16-byte core matrices the MMA reads from shared memory)
  float* scale;       // [out_dim]
  float* bias;        // [out_dim] or nullptr
  uint64_t bytes;
};

namespace goph {

// ---- device helpers -------------------------------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// 128-bit streaming load: weights are read once, keep them out of L1.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) { return __uint_as_float(b16 << 16); }

// Two packed f32 FMAs in one instruction (sm_100 fma.rn.f32x2): acc += a*b lane-wise.
__device__ __forceinline__ void fma2(float2& acc, float2 a, float2 b) {
  asm("{\n\t.reg .b64 ra, rb, rc;\n\t"
      "mov.b64 ra, {%2,%3};\n\t"
      "mov.b64 rb, {%4,%5};\n\t"
      "mov.b64 rc, {%0,%1};\n\t"
      "fma.rn.f32x2 rc, ra, rb, rc;\n\t"
      "mov.b64 {%0,%1}, rc;\n\t}"
      : "+f"(acc.x), "+f"(acc.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
}

}  // namespace goph
