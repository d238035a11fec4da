// GGUF Q8_0 and Q4_K matrices: upload (device re-layout), bit-exact dequantisation and the
// dequant-fused GEMV / small-batch projection.
//
// Replaces gemv_q8_0(_batch), gemv_q4_k(_batch), gemm_q4_raw_f32 and friends
// (backends/nvidia/ptx/q8, ptx/q4) behind GPUGGUFMatrix.ProjectBatchToBuffer,
// GemvQ4K*/GemvQ8_0* (backends/nvidia/runtime/gguf_matrix.go:121-135, q4k.go:351-595,
// q8.go:225-301).  Arithmetic specification: dequantRowQ8_0To / dequantRowQ4KTo
// (loader/gguf/quant_matrix.go:138-158, :281-329) followed by an f32 dot with x
// (model/gguf_llama.go:626-685); activations stay f32.
//
// Device layouts (same byte count as the GGUF stream, chosen so a lane's 16-byte unit is a
// run of consecutive elements with one scale):
//   Q4_K  144-byte super-block = 16-byte header {f16 d, f16 dmin, 8 x 12-bit (sc | m<<6)}
//         + 8 x 16 bytes; sub-block s in bytes [16s,16s+16), element 2i in the low nibble
//         of byte i, element 2i+1 in the high nibble.
//   Q8_0  plane of (q + 128) bytes [out][in], then f16 d [out][in/32].
//   Q5_K  176-byte super-block = the Q4_K header and nibbles (16 + 8 x 16 bytes) + 8 x 4 bytes of
//         fifth bits, bit e of sub-block s's word = element e.
//   Q6_K  four planes over the whole matrix: low nibbles [out][in/2] (element e of a 32-element
//         unit at bits 4(e%8) of word e/8), two-bit highs [out][in/4] (element e at bits 2(e%16)
//         of word e/16), int8 scales [out][in/16], f16 d [out][in/256].
#include <string.h>

#include "mlx_mma.cuh"
#include "stream_gemv.cuh"
#include "gguf_fmt.cuh"

namespace goph {

// ---- Q4_K (the streaming format policy is in gguf_fmt.cuh) ------------------------------

// GGUF super-block → device super-block, one thread per block.
__global__ void q4k_relayout_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ dst, size_t nblocks) {
  size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const uint8_t* s = raw + b * 144;
  uint8_t* o = dst + b * 144;
  o[0] = s[0];
  o[1] = s[1];
  o[2] = s[2];
  o[3] = s[3];
  const uint8_t* sc = s + 4;
  uint32_t field[8];
  for (int j = 0; j < 4; ++j) field[j] = (uint32_t)(sc[j] & 63) | ((uint32_t)(sc[j + 4] & 63) << 6);
  for (int j = 4; j < 8; ++j) {
    int k = j - 4;
    uint32_t scv = (sc[j + 4] & 0xF) | ((sc[k] >> 6) << 4);
    uint32_t mv = (sc[j + 4] >> 4) | ((sc[k + 4] >> 6) << 4);
    field[j] = scv | (mv << 6);
  }
  uint32_t words[3] = {0, 0, 0};
  for (int j = 0; j < 8; ++j) {
    int bit = 12 * j, wi = bit >> 5, sh = bit & 31;
    words[wi] |= field[j] << sh;
    if (sh > 20) words[wi + 1] |= field[j] >> (32 - sh);
  }
  for (int i = 0; i < 12; ++i) o[4 + i] = (uint8_t)(words[i >> 2] >> (8 * (i & 3)));
  const uint8_t* qs = s + 16;
  for (int sb = 0; sb < 8; ++sb) {
    const uint8_t* q = qs + (sb >> 1) * 32;
    int hi = sb & 1;
    for (int i = 0; i < 16; ++i) {
      uint8_t e0 = hi ? (q[2 * i] >> 4) : (q[2 * i] & 0xF);
      uint8_t e1 = hi ? (q[2 * i + 1] >> 4) : (q[2 * i + 1] & 0xF);
      o[16 + 16 * sb + i] = e0 | (e1 << 4);
    }
  }
}

// dequantRowQ4KTo from the device layout: (sc*d)*q - (m*dmin), every step rounded.
__global__ void q4k_dequant_kernel(const uint8_t* __restrict__ w, float* __restrict__ out, size_t nunits) {
  size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= nunits) return;
  const uint8_t* blk = w + (u >> 3) * 144;
  int s = (int)(u & 7);
  uint4 h = *reinterpret_cast<const uint4*>(blk);
  uint4 q = *reinterpret_cast<const uint4*>(blk + 16 + 16 * s);
  uint32_t f = q4k_field(h, s);
  float sd = __fmul_rn((float)(f & 63u), f16_bits_to_f32(h.x & 0xFFFFu));
  float md = __fmul_rn((float)(f >> 6), f16_bits_to_f32(h.x >> 16));
  float4* o = reinterpret_cast<float4*>(out + u * 32);
  uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __fsub_rn(__fmul_rn(sd, (float)((ws[k] >> (4 * e)) & 0xF)), md);
    o[2 * k] = make_float4(v[0], v[1], v[2], v[3]);
    o[2 * k + 1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// ---- Q8_0 (the streaming format policy is in gguf_fmt.cuh) ------------------------------

// 34-byte GGUF blocks → biased byte plane + f16 scale plane; one thread per block.
__global__ void q8_0_relayout_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ plane,
                                     uint16_t* __restrict__ d16, size_t nblocks) {
  size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const uint8_t* s = raw + b * 34;
  d16[b] = (uint16_t)(s[0] | (s[1] << 8));
  for (int i = 0; i < 32; ++i) plane[b * 32 + i] = (uint8_t)(s[2 + i] ^ 0x80);
}

// dequantRowQ8_0To from the device layout: d * float32(int8).
__global__ void q8_0_dequant_kernel(const uint8_t* __restrict__ plane, const uint16_t* __restrict__ d16,
                                    float* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float d = f16_bits_to_f32(d16[i >> 5]);
  out[i] = __fmul_rn(d, (float)((int)plane[i] - 128));
}


// ---- Q5_K ---------------------------------------------------------------------------

struct Q5KFmt {
  static constexpr int kSlots = 8;  // 32 elements per unit
  static constexpr bool kHasConsts = true;
  struct Row {
    uint4 q;
    uint32_t hb;   // fifth bits of the unit's 32 elements
    float sd, md;  // sc*d and m*dmin, each rounded to f32 as the reference does
  };
  static __device__ __forceinline__ void load(const StreamArgs& a, int row, int unit, Row& t) {
    const uint8_t* blk = a.w + (size_t)row * a.row_bytes + (size_t)(unit >> 3) * 176;
    int s = unit & 7;
    uint4 h = __ldg(reinterpret_cast<const uint4*>(blk));
    t.q = ld_stream(reinterpret_cast<const uint4*>(blk + 16 + 16 * s));
    t.hb = __ldg(reinterpret_cast<const uint32_t*>(blk + 144 + 4 * s));
    uint32_t f = q4k_field(h, s);
    t.sd = __fmul_rn((float)(f & 63u), f16_bits_to_f32(h.x & 0xFFFFu));
    t.md = __fmul_rn((float)(f >> 6), f16_bits_to_f32(h.x >> 16));
  }
  // Every five-bit value is moved to the top mantissa bits under 2^5 and reads as 32+v.
  static __device__ __forceinline__ float2 consts(float se, float so) {
    return make_float2(32.f * (se + so), se + so);
  }
  template <int M>
  static __device__ __forceinline__ void dot(const Row& t, const float4 (&xv)[M][8], const float2 (&c)[M],
                                             float (&acc)[M]) {
    float2 F[M];
#pragma unroll
    for (int m = 0; m < M; ++m) F[m] = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t w = k == 0 ? t.q.x : k == 1 ? t.q.y : k == 2 ? t.q.z : t.q.w;
      const uint32_t hb = t.hb >> (8 * k);
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t v = ((w >> (4 * e)) & 0xFu) | (((hb >> e) & 1u) << 4);
        f[e] = __uint_as_float((v << 18) | 0x42000000u);
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float4 xa = xv[m][2 * k], xb = xv[m][2 * k + 1];
        fma2(F[m], make_float2(f[0], f[1]), make_float2(xa.x, xa.y));
        fma2(F[m], make_float2(f[2], f[3]), make_float2(xa.z, xa.w));
        fma2(F[m], make_float2(f[4], f[5]), make_float2(xb.x, xb.y));
        fma2(F[m], make_float2(f[6], f[7]), make_float2(xb.z, xb.w));
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

// GGUF Q5_K super-block -> device super-block, one thread per block (loader/gguf/quant_matrix.go:331-384).
__global__ void q5k_relayout_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ dst, size_t nblocks) {
  size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const uint8_t* s = raw + b * 176;
  uint8_t* o = dst + b * 176;
  for (int i = 0; i < 4; ++i) o[i] = s[i];
  const uint8_t* sc = s + 4;
  uint32_t field[8];
  for (int j = 0; j < 4; ++j) field[j] = (uint32_t)(sc[j] & 63) | ((uint32_t)(sc[j + 4] & 63) << 6);
  for (int j = 4; j < 8; ++j) {
    int k = j - 4;
    uint32_t scv = (sc[j + 4] & 0xF) | ((sc[k] >> 6) << 4);
    uint32_t mv = (sc[j + 4] >> 4) | ((sc[k + 4] >> 6) << 4);
    field[j] = scv | (mv << 6);
  }
  uint32_t words[3] = {0, 0, 0};
  for (int j = 0; j < 8; ++j) {
    int bit = 12 * j, wi = bit >> 5, sh = bit & 31;
    words[wi] |= field[j] << sh;
    if (sh > 20) words[wi + 1] |= field[j] >> (32 - sh);
  }
  for (int i = 0; i < 12; ++i) o[4 + i] = (uint8_t)(words[i >> 2] >> (8 * (i & 3)));
  const uint8_t* qh = s + 16;
  const uint8_t* ql = s + 48;
  for (int sb = 0; sb < 8; ++sb) {
    const uint8_t* q = ql + (sb >> 1) * 32;  // sub-blocks 2g and 2g+1 share 32 bytes (low / high nibble)
    const int hi = sb & 1;
    uint32_t bits = 0;
    for (int i = 0; i < 16; ++i) {
      uint8_t e0 = hi ? (q[2 * i] >> 4) : (q[2 * i] & 0xF);
      uint8_t e1 = hi ? (q[2 * i + 1] >> 4) : (q[2 * i + 1] & 0xF);
      o[16 + 16 * sb + i] = e0 | (e1 << 4);
    }
    for (int e = 0; e < 32; ++e) bits |= (uint32_t)((qh[e] >> sb) & 1u) << e;  // bit sb of qh[e] is element e's fifth bit
    o[144 + 4 * sb + 0] = (uint8_t)bits;
    o[144 + 4 * sb + 1] = (uint8_t)(bits >> 8);
    o[144 + 4 * sb + 2] = (uint8_t)(bits >> 16);
    o[144 + 4 * sb + 3] = (uint8_t)(bits >> 24);
  }
}

// dequantRowQ5KTo from the device layout: (sc*d)*q - (m*dmin), every step rounded.
__global__ void q5k_dequant_kernel(const uint8_t* __restrict__ w, float* __restrict__ out, size_t nunits) {
  size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= nunits) return;
  const uint8_t* blk = w + (u >> 3) * 176;
  int s = (int)(u & 7);
  uint4 h = *reinterpret_cast<const uint4*>(blk);
  uint4 q = *reinterpret_cast<const uint4*>(blk + 16 + 16 * s);
  uint32_t hb = *reinterpret_cast<const uint32_t*>(blk + 144 + 4 * s);
  uint32_t f = q4k_field(h, s);
  float sd = __fmul_rn((float)(f & 63u), f16_bits_to_f32(h.x & 0xFFFFu));
  float md = __fmul_rn((float)(f >> 6), f16_bits_to_f32(h.x >> 16));
  uint32_t ws[4] = {q.x, q.y, q.z, q.w};
  for (int e = 0; e < 32; ++e) {
    uint32_t v = ((ws[e >> 3] >> (4 * (e & 7))) & 0xFu) | (((hb >> e) & 1u) << 4);
    out[u * 32 + e] = __fsub_rn(__fmul_rn(sd, (float)v), md);
  }
}

// ---- Q6_K ---------------------------------------------------------------------------

struct Q6KFmt {
  static constexpr int kSlots = 8;  // 32 elements per unit: two 16-element scale groups
  static constexpr bool kHasConsts = false;
  struct Row {
    uint4 lo;      // low nibbles
    uint2 hi;      // two-bit highs
    float m0, m1;  // d * scale of the unit's two groups, rounded to f32 as the reference does
  };
  // aux = {high plane, scale plane, d plane} packed behind the low plane: offsets in StreamArgs::bias slots
  static __device__ __forceinline__ void load(const StreamArgs& a, int row, int unit, Row& t) {
    const size_t in = (size_t)a.in_dim;
    const uint8_t* lo = a.w + (size_t)row * (in / 2) + (size_t)unit * 16;
    const uint8_t* hi = reinterpret_cast<const uint8_t*>(a.aux) + (size_t)row * (in / 4) + (size_t)unit * 8;
    const uint8_t* planes = reinterpret_cast<const uint8_t*>(a.aux) + (size_t)a.rows * (in / 4);
    const int8_t* sc = reinterpret_cast<const int8_t*>(planes) + (size_t)row * (in / 16) + (size_t)unit * 2;
    const uint16_t* dp = reinterpret_cast<const uint16_t*>(planes + (size_t)a.rows * (in / 16)) + (size_t)row * (in / 256) + (unit >> 3);
    t.lo = ld_stream(reinterpret_cast<const uint4*>(lo));
    t.hi = __ldg(reinterpret_cast<const uint2*>(hi));
    const float d = f16_bits_to_f32(__ldg(dp));
    t.m0 = __fmul_rn(d, (float)sc[0]);
    t.m1 = __fmul_rn(d, (float)sc[1]);
  }
  static __device__ __forceinline__ float2 consts(float, float) { return make_float2(0.f, 0.f); }
  template <int M>
  static __device__ __forceinline__ void dot(const Row& t, const float4 (&xv)[M][8], const float2 (&)[M], float (&acc)[M]) {
    // six-bit value v on the top mantissa bits under 2^6 reads as 64 + v; minus 96 gives v - 32
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      float2 F[M];
#pragma unroll
      for (int m = 0; m < M; ++m) F[m] = make_float2(0.f, 0.f);
      const uint32_t hw = g == 0 ? t.hi.x : t.hi.y;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const uint32_t w = g == 0 ? (k == 0 ? t.lo.x : t.lo.y) : (k == 0 ? t.lo.z : t.lo.w);
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t v = ((w >> (4 * e)) & 0xFu) | (((hw >> (2 * (8 * k + e))) & 3u) << 4);
          f[e] = __uint_as_float((v << 17) | 0x42800000u) - 96.f;
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float4 xa = xv[m][4 * g + 2 * k], xb = xv[m][4 * g + 2 * k + 1];
          fma2(F[m], make_float2(f[0], f[1]), make_float2(xa.x, xa.y));
          fma2(F[m], make_float2(f[2], f[3]), make_float2(xa.z, xa.w));
          fma2(F[m], make_float2(f[4], f[5]), make_float2(xb.x, xb.y));
          fma2(F[m], make_float2(f[6], f[7]), make_float2(xb.z, xb.w));
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) acc[m] = fmaf(g == 0 ? t.m0 : t.m1, F[m].x + F[m].y, acc[m]);
    }
  }
  static __device__ __forceinline__ float finish(const StreamArgs&, int, float v) { return v; }
};

// GGUF Q6_K super-blocks -> the four planes; one thread per (row, block) (loader/gguf/quant_matrix.go:386-426).
__global__ void q6k_relayout_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ lo, uint8_t* __restrict__ hi,
                                    int8_t* __restrict__ sc, uint16_t* __restrict__ dd, int out_dim, int in_dim) {
  const size_t nb = (size_t)in_dim / 256;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)out_dim * nb) return;
  const size_t row = idx / nb, b = idx - row * nb;
  const uint8_t* s = raw + idx * 210;
  const uint8_t* ql = s;
  const uint8_t* qh = s + 128;
  uint8_t q[256];
  int8_t scl[16];
  // element order of dequantRowQ6KTo: halves of 128; within a half l = 0..31 feeds elements l, l+32, l+64, l+96
  for (int half = 0; half < 2; ++half)
    for (int l = 0; l < 32; ++l) {
      const uint8_t a = ql[half * 64 + l], c = ql[half * 64 + l + 32], h = qh[half * 32 + l];
      q[half * 128 + l] = (a & 0x0F) | (((h >> 0) & 3) << 4);
      q[half * 128 + l + 32] = (c & 0x0F) | (((h >> 2) & 3) << 4);
      q[half * 128 + l + 64] = (a >> 4) | (((h >> 4) & 3) << 4);
      q[half * 128 + l + 96] = (c >> 4) | (((h >> 6) & 3) << 4);
    }
  // scale of element i: sc[half*8 + (l/16) + 2*quarter] with i = half*128 + quarter*32 + l -> group i/16 in order
  for (int g = 0; g < 16; ++g) {
    const int half = g / 8, quarter = (g % 8) / 2, sub = g % 2;
    scl[g] = (int8_t)s[192 + half * 8 + sub + 2 * quarter];
  }
  uint8_t* lo_o = lo + row * (in_dim / 2) + b * 128;
  uint8_t* hi_o = hi + row * (in_dim / 4) + b * 64;
  for (int w = 0; w < 32; ++w) {  // 8 elements per low word
    uint32_t v = 0;
    for (int e = 0; e < 8; ++e) v |= (uint32_t)(q[w * 8 + e] & 0xF) << (4 * e);
    for (int i = 0; i < 4; ++i) lo_o[w * 4 + i] = (uint8_t)(v >> (8 * i));
  }
  for (int w = 0; w < 16; ++w) {  // 16 elements per high word
    uint32_t v = 0;
    for (int e = 0; e < 16; ++e) v |= (uint32_t)(q[w * 16 + e] >> 4) << (2 * e);
    for (int i = 0; i < 4; ++i) hi_o[w * 4 + i] = (uint8_t)(v >> (8 * i));
  }
  for (int g = 0; g < 16; ++g) sc[row * (in_dim / 16) + b * 16 + g] = scl[g];
  dd[row * nb + b] = (uint16_t)(s[208] | (s[209] << 8));
}

// dequantRowQ6KTo from the planes: (d * scale) * (q - 32), the first product rounded to f32.
__global__ void q6k_dequant_kernel(const uint8_t* __restrict__ lo, const uint8_t* __restrict__ hi,
                                   const int8_t* __restrict__ sc, const uint16_t* __restrict__ dd,
                                   float* __restrict__ out, int out_dim, int in_dim) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)out_dim * in_dim) return;
  const size_t row = i / in_dim, col = i - row * in_dim;
  const uint32_t wl = reinterpret_cast<const uint32_t*>(lo + row * (in_dim / 2))[col / 8];
  const uint32_t wh = reinterpret_cast<const uint32_t*>(hi + row * (in_dim / 4))[col / 16];
  const int v = (int)(((wl >> (4 * (col & 7))) & 0xFu) | (((wh >> (2 * (col & 15))) & 3u) << 4)) - 32;
  const float d = f16_bits_to_f32(dd[row * (in_dim / 256) + col / 256]);
  out[i] = __fmul_rn(__fmul_rn(d, (float)sc[row * (in_dim / 16) + col / 16]), (float)v);
}

static bool valid_gguf(const goph_gguf_matrix* m) {
  return m && m->magic == kMagicGGUF && m->in_dim > 0 && m->out_dim > 0 &&
         (m->tiled || (m->data && (m->qtype == GOPH_GGUF_Q4_K || m->qtype == GOPH_GGUF_Q5_K ||
                                   ((m->qtype == GOPH_GGUF_Q8_0 || m->qtype == GOPH_GGUF_Q6_K) && m->d16))));
}

static long gguf_row_bytes(int qtype, int in_dim) {
  if (qtype == GOPH_GGUF_Q8_0) return in_dim % 32 ? -1 : (long)in_dim / 32 * 34;
  if (qtype == GOPH_GGUF_Q4_K) return in_dim % 256 ? -1 : (long)in_dim / 256 * 144;
  if (qtype == GOPH_GGUF_Q5_K) return in_dim % 256 ? -1 : (long)in_dim / 256 * 176;
  if (qtype == GOPH_GGUF_Q6_K) return in_dim % 256 ? -1 : (long)in_dim / 256 * 210;
  return -1;
}

}  // namespace goph

using namespace goph;

GOPH_API int goph_gguf_upload(int device, int qtype, const uint8_t* raw, uint64_t raw_len, int in_dim, int out_dim,
                              goph_gguf_matrix** out) {
  clear_error();
  if (!out) return fail(GOPH_E_INVALID, "goph_gguf_upload: nil result pointer");
  *out = nullptr;
  if (qtype != GOPH_GGUF_Q8_0 && qtype != GOPH_GGUF_Q4_K && qtype != GOPH_GGUF_Q5_K && qtype != GOPH_GGUF_Q6_K)
    return fail(GOPH_E_UNSUPPORTED, "GGUF quant type %d is not Q8_0, Q4_K, Q5_K or Q6_K", qtype);
  if (in_dim <= 0 || out_dim <= 0) return fail(GOPH_E_INVALID, "invalid GGUF dims in=%d out=%d", in_dim, out_dim);
  long rb = gguf_row_bytes(qtype, in_dim);
  if (rb < 0)
    return fail(GOPH_E_INVALID, "%s row n=%d not multiple of %d",
                qtype == GOPH_GGUF_Q8_0 ? "Q8_0" : qtype == GOPH_GGUF_Q4_K ? "Q4_K" : qtype == GOPH_GGUF_Q5_K ? "Q5_K" : "Q6_K", in_dim,
                qtype == GOPH_GGUF_Q8_0 ? 32 : 256);
  uint64_t need;
  if (!mul_ok((uint64_t)rb, (uint64_t)out_dim, &need)) return fail(GOPH_E_INVALID, "GGUF matrix size overflow");
  if (!raw || raw_len < need)
    return fail(GOPH_E_INVALID, "raw length=%llu, want at least %llu", (unsigned long long)raw_len,
                (unsigned long long)need);
  if (int rc = use_device(device)) return rc;

  goph_gguf_matrix* h = new goph_gguf_matrix();
  memset(h, 0, sizeof *h);
  h->magic = kMagicGGUF;
  h->device = device;
  h->qtype = qtype;
  h->in_dim = in_dim;
  h->out_dim = out_dim;
  uint8_t* tmp = nullptr;
  auto bail = [&](int rc) {
    cudaFree(tmp);
    if (rc) {
      cudaFree(h->data);
      cudaFree(h->d16);
      cudaFree(h->tiled);
      delete h;
    }
    return rc;
  };
#define UP(call)                                              \
  do {                                                        \
    cudaError_t _e = (call);                                  \
    if (_e != cudaSuccess) return bail(fail_cuda(_e, #call)); \
  } while (0)
  UP(cudaMalloc(&tmp, need));
  UP(cudaMemcpy(tmp, raw, need, cudaMemcpyHostToDevice));
  if (qtype == GOPH_GGUF_Q4_K) {
    size_t nblocks = (size_t)out_dim * (in_dim / 256);
    UP(cudaMalloc(&h->data, need));
    q4k_relayout_kernel<<<(unsigned)((nblocks + 127) / 128), 128>>>(tmp, h->data, nblocks);
    h->bytes = need;
  } else if (qtype == GOPH_GGUF_Q5_K) {
    size_t nblocks = (size_t)out_dim * (in_dim / 256);
    UP(cudaMalloc(&h->data, need));
    q5k_relayout_kernel<<<(unsigned)((nblocks + 127) / 128), 128>>>(tmp, h->data, nblocks);
    h->bytes = need;
  } else if (qtype == GOPH_GGUF_Q6_K) {
    // planes: low nibbles in data; highs, scales and d behind one another in d16
    const size_t n = (size_t)out_dim * in_dim, nblocks = n / 256;
    UP(cudaMalloc(&h->data, n / 2));
    UP(cudaMalloc(&h->d16, n / 4 + n / 16 + nblocks * 2));
    uint8_t* hi = reinterpret_cast<uint8_t*>(h->d16);
    q6k_relayout_kernel<<<(unsigned)((nblocks + 63) / 64), 64>>>(tmp, h->data, hi, reinterpret_cast<int8_t*>(hi + n / 4),
                                                                reinterpret_cast<uint16_t*>(hi + n / 4 + n / 16), out_dim, in_dim);
    h->bytes = need;
  } else {
    size_t nblocks = (size_t)out_dim * (in_dim / 32);
    UP(cudaMalloc(&h->data, nblocks * 32));
    UP(cudaMalloc(&h->d16, nblocks * 2));
    q8_0_relayout_kernel<<<(unsigned)((nblocks + 127) / 128), 128>>>(tmp, h->data, h->d16, nblocks);
    h->bytes = nblocks * 34;
  }
  UP(cudaGetLastError());
  UP(cudaDeviceSynchronize());
#undef UP
  // Large matrices go to the tensor-core layout (the CUDA-core kernels are instruction-bound on
  // this part); small ones stay in the streaming layout, whose launch is leaner.
  const bool big = (uint64_t)in_dim * (uint64_t)out_dim >= (8ull << 20);
  if (gguf_mma_supported(qtype, in_dim) && (options().gguf_layout == 2 || (options().gguf_layout == 0 && big))) {
    if (int rc = gguf_mma_make_tiled(h)) return bail(rc);
    cudaFree(h->data);
    cudaFree(h->d16);
    h->data = nullptr;
    h->d16 = nullptr;
  }
  *out = h;
  return bail(GOPH_OK);
}

GOPH_API int goph_gguf_free(goph_gguf_matrix* m) {
  clear_error();
  if (!m) return GOPH_OK;
  if (m->magic != kMagicGGUF) return fail(GOPH_E_INVALID, "goph_gguf_free: not a GGUF matrix handle");
  if (int rc = use_device(m->device)) return rc;
  cudaFree(m->data);
  cudaFree(m->d16);
  cudaFree(m->tiled);
  m->magic = 0;
  delete m;
  return GOPH_OK;
}

GOPH_API uint64_t goph_gguf_resident_bytes(const goph_gguf_matrix* m) {
  return (m && m->magic == kMagicGGUF) ? m->bytes : 0;
}

GOPH_API int goph_gguf_dequant(const goph_gguf_matrix* m, float* out_dev, uint64_t out_len, void* stream) {
  clear_error();
  if (!valid_gguf(m)) return fail(GOPH_E_INVALID, "invalid GGUF matrix handle");
  uint64_t need = (uint64_t)m->out_dim * m->in_dim;
  if (!out_dev || out_len < need)
    return fail(GOPH_E_INVALID, "dequant out length=%llu, want at least %llu", (unsigned long long)out_len,
                (unsigned long long)need);
  if ((uintptr_t)out_dev % 16) return fail(GOPH_E_INVALID, "dequant out must be 16-byte aligned");
  if (int rc = use_device(m->device)) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (m->tiled) return gguf_mma_dequant(m, out_dev, s);
  if (m->qtype == GOPH_GGUF_Q4_K) {
    size_t nunits = need / 32;
    q4k_dequant_kernel<<<(unsigned)((nunits + 255) / 256), 256, 0, s>>>(m->data, out_dev, nunits);
  } else if (m->qtype == GOPH_GGUF_Q5_K) {
    size_t nunits = need / 32;
    q5k_dequant_kernel<<<(unsigned)((nunits + 255) / 256), 256, 0, s>>>(m->data, out_dev, nunits);
  } else if (m->qtype == GOPH_GGUF_Q6_K) {
    const uint8_t* hi = reinterpret_cast<const uint8_t*>(m->d16);
    q6k_dequant_kernel<<<(unsigned)((need + 255) / 256), 256, 0, s>>>(
        m->data, hi, reinterpret_cast<const int8_t*>(hi + need / 4), reinterpret_cast<const uint16_t*>(hi + need / 4 + need / 16),
        out_dev, m->out_dim, m->in_dim);
  } else {
    q8_0_dequant_kernel<<<(unsigned)((need + 255) / 256), 256, 0, s>>>(m->data, m->d16, out_dev, need);
  }
  GOPH_CUDA(cudaGetLastError());
  return GOPH_OK;
}

GOPH_API int goph_gguf_project(float* out_dev, uint64_t out_len, const float* x_dev, uint64_t x_len, int batch,
                               const goph_gguf_matrix* m, void* stream) {
  clear_error();
  if (!valid_gguf(m)) return fail(GOPH_E_INVALID, "invalid GGUF matrix handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_x, need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)m->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)m->out_dim, &need_o))
    return fail(GOPH_E_INVALID, "batch size overflow");
  if (!x_dev || x_len < need_x || !out_dev || out_len < need_o)
    return fail(GOPH_E_INVALID, "buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len,
                (unsigned long long)need_x, (unsigned long long)out_len, (unsigned long long)need_o);
  if (int rc = use_device(m->device)) return rc;
  if (m->tiled) return gguf_mma_launch(m, out_dev, x_dev, batch, options().mlx_digits, (cudaStream_t)stream);
  StreamArgs a;
  memset(&a, 0, sizeof a);
  a.w = m->data;
  a.aux = m->d16;
  a.out = out_dev;
  a.x = x_dev;
  a.rows = m->out_dim;
  a.in_dim = m->in_dim;
  const int force_rows = options().gguf_rows;
  if (m->qtype == GOPH_GGUF_Q4_K) {
    a.units = m->in_dim / 32;
    a.row_bytes = m->in_dim / 256 * 144;
    return stream_launch<Q4KFmt>(a, m->device, batch, (cudaStream_t)stream, force_rows);
  }
  if (m->qtype == GOPH_GGUF_Q5_K) {
    a.units = m->in_dim / 32;
    a.row_bytes = m->in_dim / 256 * 176;
    return stream_launch<Q5KFmt>(a, m->device, batch, (cudaStream_t)stream, force_rows);
  }
  if (m->qtype == GOPH_GGUF_Q6_K) {
    a.units = m->in_dim / 32;
    a.row_bytes = m->in_dim / 2;
    return stream_launch<Q6KFmt>(a, m->device, batch, (cudaStream_t)stream, force_rows);
  }
  a.units = m->in_dim / 16;
  a.row_bytes = m->in_dim;
  return stream_launch<Q80Fmt>(a, m->device, batch, (cudaStream_t)stream, force_rows);
}

GOPH_API int goph_gguf_project_pair(float* out_a_dev, uint64_t out_a_len, float* out_b_dev, uint64_t out_b_len,
                                    const float* x_dev, uint64_t x_len, int batch, const goph_gguf_matrix* a,
                                    const goph_gguf_matrix* b, void* stream) {
  clear_error();
  if (!valid_gguf(a) || !valid_gguf(b)) return fail(GOPH_E_INVALID, "invalid GGUF matrix handle");
  if (a->device != b->device || a->in_dim != b->in_dim)
    return fail(GOPH_E_INVALID, "pair projection: matrices differ in device or inDim (%d vs %d)", a->in_dim, b->in_dim);
  if (a->tiled && b->tiled && a->qtype == b->qtype) {
    // both on the tensor-core path: validated like a single projection, x prepared once
    if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
    uint64_t need_x, need_a, need_b;
    if (!mul_ok((uint64_t)batch, (uint64_t)a->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)a->out_dim, &need_a) ||
        !mul_ok((uint64_t)batch, (uint64_t)b->out_dim, &need_b))
      return fail(GOPH_E_INVALID, "batch size overflow");
    if (!x_dev || x_len < need_x || !out_a_dev || out_a_len < need_a || !out_b_dev || out_b_len < need_b)
      return fail(GOPH_E_INVALID, "buffers x=%llu/%llu outA=%llu/%llu outB=%llu/%llu", (unsigned long long)x_len,
                  (unsigned long long)need_x, (unsigned long long)out_a_len, (unsigned long long)need_a,
                  (unsigned long long)out_b_len, (unsigned long long)need_b);
    if (int rc = use_device(a->device)) return rc;
    if (int rc = gguf_mma_launch(a, out_a_dev, x_dev, batch, options().mlx_digits, (cudaStream_t)stream, false)) return rc;
    return gguf_mma_launch(b, out_b_dev, x_dev, batch, options().mlx_digits, (cudaStream_t)stream, true);
  }
  if (int rc = goph_gguf_project(out_a_dev, out_a_len, x_dev, x_len, batch, a, stream)) return rc;
  return goph_gguf_project(out_b_dev, out_b_len, x_dev, x_len, batch, b, stream);
}

GOPH_API int goph_gguf_project_host(float* out_host, uint64_t out_len, const float* x_host, uint64_t x_len,
                                    int batch, const goph_gguf_matrix* m) {
  clear_error();
  if (!valid_gguf(m)) return fail(GOPH_E_INVALID, "invalid GGUF matrix handle");
  if (batch <= 0) return fail(GOPH_E_INVALID, "batch=%d", batch);
  uint64_t need_x, need_o;
  if (!mul_ok((uint64_t)batch, (uint64_t)m->in_dim, &need_x) || !mul_ok((uint64_t)batch, (uint64_t)m->out_dim, &need_o))
    return fail(GOPH_E_INVALID, "batch size overflow");
  if (!x_host || x_len < need_x || !out_host || out_len < need_o)
    return fail(GOPH_E_INVALID, "host buffers x=%llu/%llu out=%llu/%llu", (unsigned long long)x_len,
                (unsigned long long)need_x, (unsigned long long)out_len, (unsigned long long)need_o);
  if (int rc = use_device(m->device)) return rc;
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
  if (!rc) rc = goph_gguf_project(dout, need_o, dx, need_x, batch, m, nullptr);
  if (!rc) {
    e = cudaMemcpy(out_host, dout, need_o * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) rc = fail_cuda(e, "cudaMemcpy(out)");
  }
  cudaFree(dx);
  cudaFree(dout);
  return rc;
}
