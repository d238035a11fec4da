// Format policies of the streaming GEMV skeleton (stream_gemv.cuh) for GGUF Q4_K and Q8_0 matrices
// in the streaming device layouts; shared by the plain products (gguf.cu) and the work-list
// products (gguf_work.cu).
#pragma once

#include "stream_gemv.cuh"

namespace goph {

// ---- Q4_K ---------------------------------------------------------------------------

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)h));
}

// The 12-bit field of sub-block s out of the 96-bit string (y,z,w).
__device__ __forceinline__ uint32_t q4k_field(uint4 h, int s) {
  int bit = 12 * s, wi = bit >> 5, sh = bit & 31;
  uint32_t lo = wi == 0 ? h.y : wi == 1 ? h.z : h.w;
  uint32_t hi = wi == 0 ? h.z : wi == 1 ? h.w : 0u;
  return __funnelshift_r(lo, hi, sh) & 0xFFFu;
}

struct Q4KFmt {
  static constexpr int kSlots = 8;  // 32 elements per unit
  static constexpr bool kHasConsts = true;
  struct Row {
    uint4 q;
    float sd, md;  // sc*d and m*dmin, each rounded to f32 as the reference does
  };
  static __device__ __forceinline__ void load(const StreamArgs& a, int row, int unit, Row& t) {
    const uint8_t* blk = a.w + (size_t)row * a.row_bytes + (size_t)(unit >> 3) * 144;
    int s = unit & 7;
    uint4 h = __ldg(reinterpret_cast<const uint4*>(blk));
    t.q = ld_stream(reinterpret_cast<const uint4*>(blk + 16 + 16 * s));
    uint32_t f = q4k_field(h, s);
    t.sd = __fmul_rn((float)(f & 63u), f16_bits_to_f32(h.x & 0xFFFFu));
    t.md = __fmul_rn((float)(f >> 6), f16_bits_to_f32(h.x >> 16));
  }
  // Every nibble is moved to the top mantissa bits under 2^4 and reads as 16+n.
  static __device__ __forceinline__ float2 consts(float se, float so) {
    return make_float2(16.f * (se + so), se + so);
  }
  template <int M>
  static __device__ __forceinline__ void dot(const Row& t, const float4 (&xv)[M][8], const float2 (&c)[M],
                                             float (&acc)[M]) {
    float2 F[M];
#pragma unroll
    for (int m = 0; m < M; ++m) F[m] = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t w = k == 0 ? t.q.x : k == 1 ? t.q.y : k == 2 ? t.q.z : t.q.w;
      constexpr uint32_t MK = 0x00780000u, EX = 0x41800000u;
      float2 f0 = make_float2(__uint_as_float(((w << 19) & MK) | EX), __uint_as_float(((w << 15) & MK) | EX));
      float2 f1 = make_float2(__uint_as_float(((w << 11) & MK) | EX), __uint_as_float(((w << 7) & MK) | EX));
      float2 f2 = make_float2(__uint_as_float(((w << 3) & MK) | EX), __uint_as_float(((w >> 1) & MK) | EX));
      float2 f3 = make_float2(__uint_as_float(((w >> 5) & MK) | EX), __uint_as_float(((w >> 9) & MK) | EX));
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float4 xa = xv[m][2 * k], xb = xv[m][2 * k + 1];
        fma2(F[m], f0, make_float2(xa.x, xa.y));
        fma2(F[m], f1, make_float2(xa.z, xa.w));
        fma2(F[m], f2, make_float2(xb.x, xb.y));
        fma2(F[m], f3, make_float2(xb.z, xb.w));
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float d = (F[m].x + F[m].y) - c[m].x;
      acc[m] = fmaf(t.sd, d, acc[m]);
      acc[m] = fmaf(-t.md, c[m].y, acc[m]);
    }
  }
  static __device__ __forceinline__ float finish(const StreamArgs&, int, float v) { return v; }
};

// ---- Q8_0 ---------------------------------------------------------------------------

struct Q80Fmt {
  static constexpr int kSlots = 4;  // 16 elements per unit
  static constexpr bool kHasConsts = true;
  struct Row {
    uint4 q;
    float d;
  };
  static __device__ __forceinline__ void load(const StreamArgs& a, int row, int unit, Row& t) {
    t.q = ld_stream(reinterpret_cast<const uint4*>(a.w + (size_t)row * a.in_dim) + unit);
    const uint16_t* d16 = reinterpret_cast<const uint16_t*>(a.aux);
    t.d = f16_bits_to_f32(__ldg(d16 + (size_t)row * (a.in_dim / 32) + (unit >> 1)));
  }
  // A stored byte u = q+128 placed on mantissa bits 15..22 under 2^8 reads as 256+u = 384+q.
  static __device__ __forceinline__ float2 consts(float se, float so) { return make_float2(384.f * (se + so), 0.f); }
  template <int M>
  static __device__ __forceinline__ void dot(const Row& t, const float4 (&xv)[M][4], const float2 (&c)[M],
                                             float (&acc)[M]) {
    float2 F[M];
#pragma unroll
    for (int m = 0; m < M; ++m) F[m] = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t w = k == 0 ? t.q.x : k == 1 ? t.q.y : k == 2 ? t.q.z : t.q.w;
      constexpr uint32_t MK = 0x007F8000u, EX = 0x43800000u;
      float2 f0 = make_float2(__uint_as_float(((w << 15) & MK) | EX), __uint_as_float(((w << 7) & MK) | EX));
      float2 f1 = make_float2(__uint_as_float(((w >> 1) & MK) | EX), __uint_as_float(((w >> 9) & MK) | EX));
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float4 xa = xv[m][k];
        fma2(F[m], f0, make_float2(xa.x, xa.y));
        fma2(F[m], f1, make_float2(xa.z, xa.w));
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = fmaf(t.d, (F[m].x + F[m].y) - c[m].x, acc[m]);
  }
  static __device__ __forceinline__ float finish(const StreamArgs&, int, float v) { return v; }
};

}  // namespace goph
