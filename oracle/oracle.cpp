// CPU oracle for the quantized matrix-product path of rcarmo/go-pherence.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain C++, the arithmetic
// of the reference's CPU path in the reference's own evaluation order.  It is
// the checker the CUDA kernels are compared against and the timed CPU baseline;
// nothing in the shipped library links, imports or calls it.
//
// The reference is Go and no Go toolchain exists in the build image, so the
// reference itself cannot be compiled or run beside this file.  Parity of the
// restatement is pinned by re-running the reference's own known-answer and
// cross-path tests against it (tests/test_oracle_pins.py): the closed-form
// dequant/GEMV cases of backends/mlx/quant_test.go, the bit-exact
// Gemm == repeated GemvTo cases of backends/mlx/gemm_test.go, the E4M3 code
// table of backends/simd/quant/fp8/dynamic_test.go, the formula-built Q8_0 and
// Q4_K blocks of backends/nvidia/runtime/{q8,q4k}_test.go, and the MoE routing
// case of model/moe_mlx_test.go.
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -shared -fPIC  (see build.py).
// Contraction must stay off: Go on amd64 never fuses a*b+c in scalar code, and
// the AVX2 assembly the reference uses is restated with explicit fmaf().
//
// All citations are file:line inside the reference repository.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <pthread.h>

#include <condition_variable>
#include <functional>
#include <mutex>
#include <new>
#include <thread>
#include <vector>
#include <algorithm>

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------------------
// Row-parallel helper.  The reference splits rows over goroutines
// (backends/mlx/gemv.go:64-108, model/gguf_llama.go:626-672); every row is
// computed by the same scalar code whichever worker owns it, so the split
// changes timing only, never bits.
// ---------------------------------------------------------------------------
// Worker threads that live as long as the process: a GEMV of a few MB takes tens of microseconds per
// thread, less than starting the threads costs, so starting them per call (as a first version did)
// made the timed baseline slower on hosts with more cores.  One parallel region runs at a time.
class Pool {
 public:
  static Pool& get() {
    static Pool* p = make();  // never destroyed: the workers are detached and may outlive static destructors
    return *p;
  }
  // job(w) for w in [0, n): w = 0 on the calling thread, the rest on the workers
  void run(int n, const std::function<void(int)>& job) {
    std::lock_guard<std::mutex> region(region_mu_);
    {
      std::lock_guard<std::mutex> l(mu_);
      while (workers_ < n - 1) {
        std::thread([this] { work(); }).detach();
        ++workers_;
      }
      job_ = &job;
      next_ = 1;
      total_ = n;
      pending_ = n - 1;
    }
    cv_.notify_all();
    job(0);
    std::unique_lock<std::mutex> l(mu_);
    done_.wait(l, [&] { return pending_ == 0; });
    job_ = nullptr;
  }

 private:
  static Pool* make() {
    Pool* p = new Pool;
    // a forked child has none of the parent's threads: it starts its own pool on first use
    pthread_atfork(nullptr, nullptr, [] { new (&Pool::get()) Pool; });
    return p;
  }
  void work() {
    for (;;) {
      std::unique_lock<std::mutex> l(mu_);
      cv_.wait(l, [&] { return job_ && next_ < total_; });
      const int w = next_++;
      const std::function<void(int)>* job = job_;
      l.unlock();
      (*job)(w);
      l.lock();
      if (--pending_ == 0) done_.notify_one();
    }
  }
  std::mutex region_mu_, mu_;
  std::condition_variable cv_, done_;
  const std::function<void(int)>* job_ = nullptr;
  int workers_ = 0, next_ = 0, total_ = 0, pending_ = 0;
};

template <class F>
void parallel_rows(int rows, int nthreads, F&& fn) {
  if (nthreads <= 1 || rows < 2) {
    fn(0, rows);
    return;
  }
  if (nthreads > rows) nthreads = rows;
  const int chunk = (rows + nthreads - 1) / nthreads;
  const int parts = (rows + chunk - 1) / chunk;
  const std::function<void(int)> job = [&](int w) {
    const int r0 = w * chunk, r1 = std::min(rows, r0 + chunk);
    if (r0 < r1) fn(r0, r1);
  };
  Pool::get().run(parts, job);
}

// half/half.go:75-96 — IEEE half to float, subnormals normalised by shifting.
float f16_to_f32(uint16_t u) {
  uint32_t sign = u >> 15, exp = (u >> 10) & 0x1F, mant = u & 0x3FF, bits;
  if (exp == 0x1F) {
    bits = sign << 31 | 0x7F800000u | mant << 13;
  } else {
    if (exp == 0) {
      if (mant == 0) {
        bits = sign << 31;
        float f;
        std::memcpy(&f, &bits, 4);
        return f;
      }
      while ((mant & 0x400) == 0) {
        mant <<= 1;
        exp--;
      }
      exp++;
      mant &= 0x3FF;
    }
    bits = sign << 31 | (exp + 112) << 23 | mant << 13;
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// ---------------------------------------------------------------------------
// MLX affine quantisation (backends/mlx).
// ---------------------------------------------------------------------------

// backends/mlx/validate.go:9-41 — returns 0 when the descriptor is well formed.
int mlx_validate(long w_len, long s_len, long b_len, int out_dim, int in_dim,
                 int gs, int groups, int bits) {
  if (bits <= 0 || bits > 32 || 32 % bits != 0) return 1;
  if (out_dim <= 0 || in_dim <= 0 || gs <= 0 || groups <= 0) return 2;
  int pf = 32 / bits;
  if (in_dim % pf != 0) return 3;
  if (in_dim % gs != 0 || groups != in_dim / gs) return 4;
  long want_w = (long)out_dim * (in_dim / pf);
  long want_s = (long)out_dim * groups;
  if (w_len < want_w) return 5;
  if (s_len < want_s || b_len < want_s) return 6;
  return 0;
}

// backends/mlx/dequant.go:95-118 — out = float32(nibble)*scale + bias, the
// product rounded to f32 before the add (two roundings).
void mlx_dequant_rows(float* out, const uint32_t* w, const float* sc,
                      const float* bi, int in_dim, int gs, int bits, int r0,
                      int r1) {
  int pf = 32 / bits, groups = in_dim / gs;
  uint32_t mask = bits == 32 ? 0xFFFFFFFFu : ((1u << bits) - 1);
  for (int row = r0; row < r1; ++row) {
    const uint32_t* wr = w + (size_t)row * (in_dim / pf);
    const float* s = sc + (size_t)row * groups;
    const float* b = bi + (size_t)row * groups;
    float* o = out + (size_t)row * in_dim;
    for (int g = 0; g < groups; ++g) {
      float scale = s[g], bias = b[g];
      for (int e = 0; e < gs; ++e) {
        int idx = g * gs + e;
        uint32_t v = (wr[idx / pf] >> ((idx % pf) * bits)) & mask;
        float p = (float)v * scale;
        o[idx] = p + bias;
      }
    }
  }
}

// backends/mlx/gemv.go:147-158 — per-group sums of x, eight values added
// left to right and then added to the running group sum.
void mlx_xsums(const float* x, int groups, int gs, float* dst) {
  int ppg = gs / 8;
  for (int g = 0; g < groups; ++g) {
    const float* xb = x + (size_t)g * gs;
    float xsum = 0.f;
    for (int p = 0; p < ppg; ++p) {
      const float* xi = xb + p * 8;
      float t = xi[0] + xi[1];
      t = t + xi[2];
      t = t + xi[3];
      t = t + xi[4];
      t = t + xi[5];
      t = t + xi[6];
      t = t + xi[7];
      xsum = xsum + t;
    }
    dst[g] = xsum;
  }
}

// backends/mlx/gemv.go:178-209 (and gemm.go:140-306, whose per-batch-row
// arithmetic is the same expression): for each group, eight products are added
// left to right, that partial is added to gsum, and the row sum takes
// gsum*scale + xsum[g]*bias (each product rounded, then added, then added).
inline float mlx4_row(const uint32_t* wr, const float* s, const float* b,
                      const float* x, const float* xsum, int groups, int gs) {
  int ppg = gs / 8;
  float sum = 0.f;
  for (int g = 0; g < groups; ++g) {
    const uint32_t* pk = wr + g * ppg;
    const float* xb = x + (size_t)g * gs;
    float gsum = 0.f;
    for (int p = 0; p < ppg; ++p) {
      uint32_t q = pk[p];
      const float* xi = xb + p * 8;
      float t = (float)(q & 0xF) * xi[0];
      t = t + (float)((q >> 4) & 0xF) * xi[1];
      t = t + (float)((q >> 8) & 0xF) * xi[2];
      t = t + (float)((q >> 12) & 0xF) * xi[3];
      t = t + (float)((q >> 16) & 0xF) * xi[4];
      t = t + (float)((q >> 20) & 0xF) * xi[5];
      t = t + (float)((q >> 24) & 0xF) * xi[6];
      t = t + (float)((q >> 28) & 0xF) * xi[7];
      gsum = gsum + t;
    }
    float a = gsum * s[g];
    float c = xsum[g] * b[g];
    sum = sum + (a + c);
  }
  return sum;
}

// backends/mlx/gemv.go:116-144 — generic-bit-width row (used when bits != 4 or
// the group size is not a multiple of 8).
inline float mlx_generic_row(const uint32_t* wr, const float* s, const float* b,
                             const float* x, int groups, int gs, int bits) {
  int pf = 32 / bits;
  uint32_t mask = bits == 32 ? 0xFFFFFFFFu : ((1u << bits) - 1);
  float sum = 0.f;
  for (int g = 0; g < groups; ++g) {
    float gsum = 0.f, xsum = 0.f;
    for (int e = 0; e < gs; ++e) {
      int idx = g * gs + e;
      float v = (float)((wr[idx / pf] >> ((idx % pf) * bits)) & mask);
      gsum = gsum + v * x[idx];
      xsum = xsum + x[idx];
    }
    float a = gsum * s[g];
    float c = xsum * b[g];
    sum = sum + (a + c);
  }
  return sum;
}

void mlx_gemv_impl(float* out, const float* x, const uint32_t* w,
                   const float* sc, const float* bi, int out_dim, int in_dim,
                   int gs, int bits, int nthreads) {
  int groups = in_dim / gs;
  bool four = bits == 4 && gs % 8 == 0;  // gemv.go:18
  std::vector<float> xsum;
  if (four) {
    xsum.resize(groups);
    mlx_xsums(x, groups, gs, xsum.data());
  }
  int pf = 32 / bits;
  parallel_rows(out_dim, nthreads, [&](int r0, int r1) {
    for (int r = r0; r < r1; ++r) {
      const uint32_t* wr = w + (size_t)r * (in_dim / pf);
      const float* s = sc + (size_t)r * groups;
      const float* b = bi + (size_t)r * groups;
      out[r] = four ? mlx4_row(wr, s, b, x, xsum.data(), groups, gs)
                    : mlx_generic_row(wr, s, b, x, groups, gs, bits);
    }
  });
}

// ---------------------------------------------------------------------------
// GGUF block formats (loader/gguf/quant_matrix.go).
// ---------------------------------------------------------------------------

// quant_matrix.go:138-158 — 34-byte block: f16 d, 32 int8; w = d*float32(q).
void q8_0_dequant_row(float* dst, const uint8_t* raw, int n) {
  int nb = n / 32;
  for (int b = 0; b < nb; ++b) {
    const uint8_t* blk = raw + (size_t)b * 34;
    float d = f16_to_f32((uint16_t)(blk[0] | blk[1] << 8));
    for (int i = 0; i < 32; ++i) dst[b * 32 + i] = d * (float)(int8_t)blk[2 + i];
  }
}

// quant_matrix.go:281-329 — 144-byte super-block: f16 d, f16 dmin, 12 bytes of
// 6-bit scales/mins, 128 quant bytes.  Sub-blocks 2j and 2j+1 share bytes
// qs[32j..32j+32) (low nibbles, then high nibbles).  w = (sc*d)*q - (m*dmin),
// with sc*d and m*dmin each rounded to f32 first.
void q4k_dequant_row(float* dst, const uint8_t* raw, int n) {
  int nb = n / 256;
  for (int b = 0; b < nb; ++b) {
    const uint8_t* blk = raw + (size_t)b * 144;
    float d = f16_to_f32((uint16_t)(blk[0] | blk[1] << 8));
    float dmin = f16_to_f32((uint16_t)(blk[2] | blk[3] << 8));
    const uint8_t* sc = blk + 4;
    const uint8_t* qs = blk + 16;
    float scales[8], mins[8];
    for (int j = 0; j < 4; ++j) {
      scales[j] = (float)(sc[j] & 63) * d;
      mins[j] = (float)(sc[j + 4] & 63) * dmin;
    }
    for (int j = 4; j < 8; ++j) {
      int k = j - 4;
      scales[j] = (float)((sc[j + 4] & 0xF) | ((sc[k] >> 6) << 4)) * d;
      mins[j] = (float)((sc[j + 4] >> 4) | ((sc[k + 4] >> 6) << 4)) * dmin;
    }
    float* o = dst + (size_t)b * 256;
    for (int group = 0; group < 8; ++group) {
      const uint8_t* q = qs + (group / 2) * 32;
      for (int i = 0; i < 16; ++i) {
        int q0, q1;
        if (group % 2 == 0) {
          q0 = q[i] & 0x0F;
          q1 = q[i + 16] & 0x0F;
        } else {
          q0 = q[i] >> 4;
          q1 = q[i + 16] >> 4;
        }
        float p0 = scales[group] * (float)q0;
        float p1 = scales[group] * (float)q1;
        o[group * 32 + i] = p0 - mins[group];
        o[group * 32 + 16 + i] = p1 - mins[group];
      }
    }
  }
}

// loader/gguf/quant_matrix.go:331-384 — Q5_K: 176-byte super-blocks {f16 d, f16 dmin, 12 scale
// bytes (the Q4_K packing), 32 bytes of fifth bits, 128 bytes of low nibbles}; groups of 64
// elements share 32 nibble bytes (low / high nibble) and two bits of each qh byte.
void q5k_dequant_row(float* dst, const uint8_t* raw, int n) {
  for (int b = 0; b < n / 256; ++b) {
    const uint8_t* blk = raw + (size_t)b * 176;
    float d = f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    float dmin = f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
    const uint8_t* sc = blk + 4;
    const uint8_t* qh = blk + 16;
    const uint8_t* ql = blk + 48;
    float scales[8], mins[8];
    for (int j = 0; j < 4; ++j) {
      scales[j] = (float)(sc[j] & 63) * d;
      mins[j] = (float)(sc[j + 4] & 63) * dmin;
    }
    for (int j = 4; j < 8; ++j) {
      int k = j - 4;
      scales[j] = (float)((sc[j + 4] & 0x0f) | ((sc[k] >> 6) << 4)) * d;
      mins[j] = (float)((sc[j + 4] >> 4) | ((sc[k + 4] >> 6) << 4)) * dmin;
    }
    int is = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int group = 0; group < 4; ++group) {
      float d1 = scales[is], m1 = mins[is], d2 = scales[is + 1], m2 = mins[is + 1];
      for (int i = 0; i < 32; ++i) {
        int q1 = ql[i] & 0x0f;
        if (qh[i] & u1) q1 += 16;
        int q2 = ql[i] >> 4;
        if (qh[i] & u2) q2 += 16;
        dst[b * 256 + group * 64 + i] = d1 * (float)q1 - m1;
        dst[b * 256 + group * 64 + 32 + i] = d2 * (float)q2 - m2;
      }
      ql += 32;
      is += 2;
      u1 = (uint8_t)(u1 << 2);
      u2 = (uint8_t)(u2 << 2);
    }
  }
}

// loader/gguf/quant_matrix.go:386-426 — Q6_K: 210-byte super-blocks {128 bytes of low nibbles,
// 64 bytes of two-bit highs, 16 int8 scales, f16 d}; value = d * scale * (q - 32), the product
// d * scale rounded to f32 first.
void q6k_dequant_row(float* dst, const uint8_t* raw, int n) {
  for (int b = 0; b < n / 256; ++b) {
    const uint8_t* blk = raw + (size_t)b * 210;
    const uint8_t* ql = blk;
    const uint8_t* qh = blk + 128;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192);
    float d = f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
    float* y = dst + (size_t)b * 256;
    for (int half = 0; half < 2; ++half) {
      for (int l = 0; l < 32; ++l) {
        int is = l / 16;
        int q1 = (int8_t)((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
        int q2 = (int8_t)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
        int q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
        int q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
        y[l] = d * (float)sc[is + 0] * (float)q1;
        y[l + 32] = d * (float)sc[is + 2] * (float)q2;
        y[l + 64] = d * (float)sc[is + 4] * (float)q3;
        y[l + 96] = d * (float)sc[is + 6] * (float)q4;
      }
      y += 128;
      ql += 64;
      qh += 32;
      sc += 8;
    }
  }
}

enum { GGUF_Q8_0 = 8, GGUF_Q4_K = 12, GGUF_Q5_K = 13, GGUF_Q6_K = 14 };  // ggml type ids (loader/gguf/gguf.go:51-56)

int gguf_row_bytes(int qtype, int in_dim) {
  if (qtype == GGUF_Q8_0) return in_dim % 32 ? -1 : in_dim / 32 * 34;
  if (qtype == GGUF_Q4_K) return in_dim % 256 ? -1 : in_dim / 256 * 144;
  if (qtype == GGUF_Q5_K) return in_dim % 256 ? -1 : in_dim / 256 * 176;
  if (qtype == GGUF_Q6_K) return in_dim % 256 ? -1 : in_dim / 256 * 210;
  return -1;
}

void gguf_dequant_row(float* dst, const uint8_t* raw, int qtype, int n) {
  if (qtype == GGUF_Q8_0)
    q8_0_dequant_row(dst, raw, n);
  else if (qtype == GGUF_Q5_K)
    q5k_dequant_row(dst, raw, n);
  else if (qtype == GGUF_Q6_K)
    q6k_dequant_row(dst, raw, n);
  else
    q4k_dequant_row(dst, raw, n);
}

// model/gguf_llama.go:675-681 — sequential f32 dot, product rounded then added.
inline float dot_f32_seq(const float* a, const float* b, int n) {
  float sum = 0.f;
  for (int i = 0; i < n; ++i) sum = sum + a[i] * b[i];
  return sum;
}

// ---------------------------------------------------------------------------
// FP8 E4M3FN (backends/simd/quant/fp8).
// ---------------------------------------------------------------------------

// fp8.go:85-106 — bias 7, subnormals at exponent 0, 0x7f/0xff are NaN.
float e4m3_decode(uint8_t code) {
  int sign = code & 0x80, exp = (code >> 3) & 0x0F, mant = code & 0x07;
  float v;
  if (exp == 0) {
    v = mant == 0 ? 0.f : (float)mant / 8 * (float)std::ldexp(1.0, -6);
  } else if (exp == 0x0F && mant == 0x07) {
    v = std::nanf("");
  } else {
    v = (1 + (float)mant / 8) * (float)std::ldexp(1.0, exp - 7);
  }
  return sign ? -v : v;
}

struct E4M3Table {
  float v[256];
  E4M3Table() {
    for (int i = 0; i < 256; ++i) v[i] = e4m3_decode((uint8_t)i);
  }
};
const E4M3Table& e4m3_lut() {
  static E4M3Table t;
  return t;
}

// The horizontal reduction every AVX2 dot in the reference ends with:
// vextractf128+vaddps, then vhaddps twice
// (backends/simd/quant/fp8/dot_amd64.s:44-49, backends/simd/runtime/simd_amd64.s:42-46).
inline float hsum8(const float* a) {
  float b0 = a[0] + a[4], b1 = a[1] + a[5], b2 = a[2] + a[6], b3 = a[3] + a[7];
  float c0 = b0 + b1, c1 = b2 + b3;
  return c0 + c1;
}

// dot_amd64.s:17-63 — one 8-lane FMA accumulator over blocks of 8, horizontal
// reduce, then a scalar FMA tail.  acc lane j holds sum over blocks of
// fma(x, lut[w], acc).
float fp8_dot_avx2(const float* x, const uint8_t* w, int n) {
  const float* lut = e4m3_lut().v;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = 0;
  for (; i + 8 <= n; i += 8)
    for (int j = 0; j < 8; ++j) acc[j] = std::fmaf(x[i + j], lut[w[i + j]], acc[j]);
  float r = hsum8(acc);
  for (; i < n; ++i) r = std::fmaf(x[i], lut[w[i]], r);
  return r;
}

// fp8.go:200-206 — the scalar fallback (hosts without AVX2+FMA).
float fp8_dot_scalar(const float* x, const uint8_t* w, int n) {
  const float* lut = e4m3_lut().v;
  float acc = 0.f;
  for (int j = 0; j < n; ++j) acc = acc + lut[w[j]] * x[j];
  return acc;
}

// simd_amd64.s:6-78 — Sdot: two 8-lane FMA accumulators over strides of 16,
// acc0 += acc1, optional 8-wide step into acc0, horizontal reduce, a 4-wide
// tail reduced on its own and added, then a scalar FMA tail.
float sdot_avx2(const float* x, const float* y, int n) {
  float a0[8] = {0}, a1[8] = {0};
  int i = 0;
  for (; i + 16 <= n; i += 16)
    for (int j = 0; j < 8; ++j) {
      a0[j] = std::fmaf(x[i + j], y[i + j], a0[j]);
      a1[j] = std::fmaf(x[i + 8 + j], y[i + 8 + j], a1[j]);
    }
  for (int j = 0; j < 8; ++j) a0[j] = a0[j] + a1[j];
  if (n - i >= 8) {
    for (int j = 0; j < 8; ++j) a0[j] = std::fmaf(x[i + j], y[i + j], a0[j]);
    i += 8;
  }
  float r = hsum8(a0);
  if (n - i >= 4) {
    float t[4];
    for (int j = 0; j < 4; ++j) t[j] = std::fmaf(y[i + j], x[i + j], 0.f);
    float u0 = t[0] + t[1], u1 = t[2] + t[3];
    r = r + (u0 + u1);
    i += 4;
  }
  for (; i < n; ++i) r = std::fmaf(y[i], x[i], r);
  return r;
}

// simd_amd64.s:148-225 — Sdotx4 (len%16==0 only): per activation row two 8-lane
// accumulators, acc_a += acc_b, horizontal reduce.
void sdotx4_avx2(const float* w, const float* x, int stride, int n, float d[4]) {
  for (int r = 0; r < 4; ++r) {
    const float* xr = x + (size_t)r * stride;
    float a0[8] = {0}, a1[8] = {0};
    for (int i = 0; i < n; i += 16)
      for (int j = 0; j < 8; ++j) {
        a0[j] = std::fmaf(w[i + j], xr[i + j], a0[j]);
        a1[j] = std::fmaf(w[i + 8 + j], xr[i + 8 + j], a1[j]);
      }
    for (int j = 0; j < 8; ++j) a0[j] = a0[j] + a1[j];
    d[r] = hsum8(a0);
  }
}

// sdotx4.go:16-30 — scalar fallback for lengths not divisible by 16.
void sdotx4_scalar(const float* w, const float* x, int stride, int n, float d[4]) {
  d[0] = d[1] = d[2] = d[3] = 0.f;
  for (int i = 0; i < n; ++i)
    for (int r = 0; r < 4; ++r) d[r] = d[r] + w[i] * x[(size_t)r * stride + i];
}

}  // namespace

// ===========================================================================
// C ABI (ctypes).  Return 0 on success; non-zero mirrors the reference's
// "false"/error for malformed input and writes nothing.
// ===========================================================================

ORC_API float orc_f16_to_f32(uint16_t u) { return f16_to_f32(u); }

// backends/mlx/f16.go / load.go:139-157 — bf16 widening is a 16-bit shift.
ORC_API float orc_bf16_to_f32(uint16_t u) {
  uint32_t b = (uint32_t)u << 16;
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}

ORC_API int orc_mlx_validate(long w_len, long s_len, long b_len, int out_dim,
                             int in_dim, int gs, int groups, int bits) {
  return mlx_validate(w_len, s_len, b_len, out_dim, in_dim, gs, groups, bits);
}

// mlx.DequantTo (backends/mlx/dequant.go:30-42).
ORC_API int orc_mlx_dequant(float* out, long out_len, const uint32_t* w, long w_len,
                            const float* sc, const float* bi, long s_len,
                            int out_dim, int in_dim, int gs, int bits, int nthreads) {
  if (gs <= 0 || mlx_validate(w_len, s_len, s_len, out_dim, in_dim, gs, in_dim / gs, bits))
    return 1;
  if (out_len < (long)out_dim * in_dim) return 2;
  parallel_rows(out_dim, nthreads, [&](int r0, int r1) {
    mlx_dequant_rows(out, w, sc, bi, in_dim, gs, bits, r0, r1);
  });
  return 0;
}

// mlx.GemvTo / GemvParallel (backends/mlx/gemv.go:14-27, :64-108).
ORC_API int orc_mlx_gemv(float* out, long out_len, const float* x, long x_len,
                         const uint32_t* w, long w_len, const float* sc,
                         const float* bi, long s_len, int out_dim, int in_dim,
                         int gs, int bits, int nthreads) {
  if (gs <= 0 || mlx_validate(w_len, s_len, s_len, out_dim, in_dim, gs, in_dim / gs, bits))
    return 1;
  if (out_len < out_dim || x_len < in_dim) return 2;
  mlx_gemv_impl(out, x, w, sc, bi, out_dim, in_dim, gs, bits, nthreads);
  return 0;
}

// mlx.Gemm (backends/mlx/gemm.go:21-37): x [batch,in], out [batch,out].
// Batches are walked in tiles of four (gemm.go:83-97); a tile of one falls
// back to GemvTo, tiles of 2..4 share each unpacked word across the tile
// (gemm.go:140-306).  Per batch row the expression is mlx4_row, so a tile is
// restated as its rows.
ORC_API int orc_mlx_gemm(float* out, long out_len, const float* x, long x_len,
                         int batch, const uint32_t* w, long w_len, const float* sc,
                         const float* bi, long s_len, int out_dim, int in_dim,
                         int gs, int bits, int nthreads) {
  if (batch <= 0 || gs <= 0 ||
      mlx_validate(w_len, s_len, s_len, out_dim, in_dim, gs, in_dim / gs, bits))
    return 1;
  if (x_len < (long)batch * in_dim || out_len < (long)batch * out_dim) return 2;
  for (int b = 0; b < batch; ++b)
    mlx_gemv_impl(out + (size_t)b * out_dim, x + (size_t)b * in_dim, w, sc, bi,
                  out_dim, in_dim, gs, bits, nthreads);
  return 0;
}

ORC_API int orc_gguf_row_bytes(int qtype, int in_dim) { return gguf_row_bytes(qtype, in_dim); }

// QuantMatrix.DequantRowTo over every row (loader/gguf/quant_matrix.go:42-60).
ORC_API int orc_gguf_dequant(float* out, long out_len, const uint8_t* raw, long raw_len,
                             int qtype, int in_dim, int out_dim, int nthreads) {
  int rb = gguf_row_bytes(qtype, in_dim);
  if (rb < 0 || out_dim <= 0) return 1;
  if (raw_len < (long)rb * out_dim || out_len < (long)in_dim * out_dim) return 2;
  parallel_rows(out_dim, nthreads, [&](int r0, int r1) {
    for (int r = r0; r < r1; ++r)
      gguf_dequant_row(out + (size_t)r * in_dim, raw + (size_t)r * rb, qtype, in_dim);
  });
  return 0;
}

// gemvGGUFQuantRowsPureGo (model/gguf_llama.go:626-672): dequantise a row into
// scratch, then a sequential f32 dot with x.  batch>1 repeats it per x row.
ORC_API int orc_gguf_gemv(float* out, long out_len, const float* x, long x_len, int batch,
                          const uint8_t* raw, long raw_len, int qtype, int in_dim,
                          int out_dim, int nthreads) {
  int rb = gguf_row_bytes(qtype, in_dim);
  if (rb < 0 || out_dim <= 0 || batch <= 0) return 1;
  if (raw_len < (long)rb * out_dim || out_len < (long)batch * out_dim ||
      x_len < (long)batch * in_dim)
    return 2;
  parallel_rows(out_dim, nthreads, [&](int r0, int r1) {
    std::vector<float> row(in_dim);
    for (int r = r0; r < r1; ++r) {
      gguf_dequant_row(row.data(), raw + (size_t)r * rb, qtype, in_dim);
      for (int b = 0; b < batch; ++b)
        out[(size_t)b * out_dim + r] = dot_f32_seq(row.data(), x + (size_t)b * in_dim, in_dim);
    }
  });
  return 0;
}

// ---------------------------------------------------------------------------
// GPTQ symmetric INT4 (backends/simd/quant/q4): qweight [in/8][out] int32 (input 8p+k in bits
// 4k..4k+3 of row p), g_idx [in], scales [groups][out]; weight = scale * (q - 8).
// ---------------------------------------------------------------------------

// validate.go:32-75 — dims, lengths, g_idx non-negative, scales cover max(g_idx)+1 groups.
int gptq_validate_sym(long qw_len, const int32_t* gidx, long g_len, long s_len, int in_dim, int out_dim) {
  if (in_dim <= 0 || out_dim <= 0 || in_dim % 8 != 0) return 1;
  if (qw_len < (long)(in_dim / 8) * out_dim || g_len < in_dim) return 2;
  int max_group = -1;
  for (int i = 0; i < in_dim; ++i) {
    if (gidx[i] < 0) return 3;
    if (gidx[i] > max_group) max_group = gidx[i];
  }
  if (s_len < (long)(max_group + 1) * out_dim) return 4;
  return 0;
}

// dequant.go:181-197 — out[j*in + i] = scale[g(i)][j] * float32(q - 8).
ORC_API int orc_gptq_dequant_sym(float* out, long out_len, const int32_t* qw, long qw_len, const int32_t* gidx,
                                 long g_len, const float* sc, long s_len, int in_dim, int out_dim) {
  if (int rc = gptq_validate_sym(qw_len, gidx, g_len, s_len, in_dim, out_dim)) return rc;
  if (out_len < (long)in_dim * out_dim) return 5;
  for (int p = 0; p < in_dim / 8; ++p)
    for (int bit = 0; bit < 8; ++bit) {
      int i = p * 8 + bit;
      const float* srow = sc + (size_t)gidx[i] * out_dim;
      for (int j = 0; j < out_dim; ++j) {
        int q = (int)(((uint32_t)qw[(size_t)p * out_dim + j] >> (4 * bit)) & 0xF);
        out[(size_t)j * in_dim + i] = srow[j] * (float)(q - 8);
      }
    }
  return 0;
}

// gemv.go:76-94 and gemm_sym_portable.go:7-150 — activation rows in tiles of up to four; a tile of
// one adds (x*scale)*(q-8), larger tiles form w = scale*(q-8) once and add x*w per row.
ORC_API int orc_gptq_gemm_sym(float* out, long out_len, const float* x, long x_len, int batch, const int32_t* qw,
                              long qw_len, const int32_t* gidx, long g_len, const float* sc, long s_len, int in_dim,
                              int out_dim) {
  if (int rc = gptq_validate_sym(qw_len, gidx, g_len, s_len, in_dim, out_dim)) return rc;
  if (batch <= 0 || out_len < (long)batch * out_dim || x_len < (long)batch * in_dim) return 5;
  for (long k = 0; k < (long)batch * out_dim; ++k) out[k] = 0.f;
  for (int b = 0; b < batch; b += 4) {
    int rem = std::min(4, batch - b);
    for (int p = 0; p < in_dim / 8; ++p)
      for (int bit = 0; bit < 8; ++bit) {
        int i = p * 8 + bit;
        const float* srow = sc + (size_t)gidx[i] * out_dim;
        for (int j = 0; j < out_dim; ++j) {
          float q = (float)((int)(((uint32_t)qw[(size_t)p * out_dim + j] >> (4 * bit)) & 0xF) - 8);
          if (rem == 1) {
            float xs = x[(size_t)b * in_dim + i] * srow[j];
            out[(size_t)b * out_dim + j] += xs * q;
          } else {
            float wv = srow[j] * q;
            for (int r = 0; r < rem; ++r) out[(size_t)(b + r) * out_dim + j] += x[(size_t)(b + r) * in_dim + i] * wv;
          }
        }
      }
  }
  return 0;
}

ORC_API float orc_e4m3_decode(uint8_t code) { return e4m3_decode(code); }

// Linear.DequantRowTo over all rows (fp8.go:181-198): lut[w]*scale.
ORC_API int orc_fp8_dequant(float* out, const uint8_t* w, const float* scale, int scale_len,
                            int out_dim, int in_dim) {
  if (out_dim <= 0 || in_dim <= 0 || (scale_len != 1 && scale_len != out_dim)) return 1;
  const float* lut = e4m3_lut().v;
  for (int r = 0; r < out_dim; ++r) {
    float s = scale_len == 1 ? scale[0] : scale[r];
    for (int j = 0; j < in_dim; ++j)
      out[(size_t)r * in_dim + j] = lut[w[(size_t)r * in_dim + j]] * s;
  }
  return 0;
}

// Linear.GemvTo (fp8.go:219-239): out[r] = dot(x, W[r])*scale[r] (+ bias[r]).
// avx2 != 0 selects the amd64 AVX2+FMA evaluation order (dot_amd64.go:13-18),
// 0 the scalar fallback.
ORC_API int orc_fp8_gemv(float* out, const float* x, const uint8_t* w, const float* scale,
                         int scale_len, const float* bias, int out_dim, int in_dim,
                         int avx2, int nthreads) {
  if (out_dim <= 0 || in_dim <= 0 || (scale_len != 1 && scale_len != out_dim)) return 1;
  parallel_rows(out_dim, nthreads, [&](int r0, int r1) {
    for (int r = r0; r < r1; ++r) {
      float s = scale_len == 1 ? scale[0] : scale[r];
      const uint8_t* wr = w + (size_t)r * in_dim;
      float acc = avx2 ? fp8_dot_avx2(x, wr, in_dim) : fp8_dot_scalar(x, wr, in_dim);
      float o = acc * s;
      if (bias) o = o + bias[r];
      out[r] = o;
    }
  });
  return 0;
}

// Linear.BatchGemvTo (batch.go:56-87, :177-207): batch 1 is GemvTo's loop;
// batch > 1 dequantises each row once WITH the scale folded in, then Sdotx4
// over groups of four activation rows and Sdot over the remainder, + bias.
ORC_API int orc_fp8_batch_gemv(float* out, const float* x, int batch, const uint8_t* w,
                               const float* scale, int scale_len, const float* bias,
                               int out_dim, int in_dim, int avx2, int nthreads) {
  if (out_dim <= 0 || in_dim <= 0 || (scale_len != 1 && scale_len != out_dim)) return 1;
  if (batch <= 0) return 0;
  if (batch == 1)
    return orc_fp8_gemv(out, x, w, scale, scale_len, bias, out_dim, in_dim, avx2, nthreads);
  const float* lut = e4m3_lut().v;
  parallel_rows(out_dim, nthreads, [&](int r0, int r1) {
    std::vector<float> wf(in_dim);
    for (int r = r0; r < r1; ++r) {
      float s = scale_len == 1 ? scale[0] : scale[r];
      const uint8_t* wr = w + (size_t)r * in_dim;
      for (int j = 0; j < in_dim; ++j) wf[j] = lut[wr[j]] * s;
      float bz = bias ? bias[r] : 0.f;
      int b = 0;
      for (; b + 4 <= batch; b += 4) {
        float d[4];
        if (avx2 && in_dim % 16 == 0)
          sdotx4_avx2(wf.data(), x + (size_t)b * in_dim, in_dim, in_dim, d);
        else
          sdotx4_scalar(wf.data(), x + (size_t)b * in_dim, in_dim, in_dim, d);
        for (int k = 0; k < 4; ++k) out[(size_t)(b + k) * out_dim + r] = d[k] + bz;
      }
      for (; b < batch; ++b) {
        const float* xr = x + (size_t)b * in_dim;
        float d = avx2 ? sdot_avx2(wf.data(), xr, in_dim) : dot_f32_seq(wf.data(), xr, in_dim);
        out[(size_t)b * out_dim + r] = d + bz;
      }
    }
  });
  return 0;
}

// simd.SoftmaxInPlace (backends/simd/runtime/softmax.go:9-30).
ORC_API int orc_softmax(float* x, int n) {
  if (n <= 0) return 1;
  float mx = x[0];
  for (int i = 1; i < n; ++i)
    if (x[i] > mx) mx = x[i];
  float sum = 0.f;
  for (int i = 0; i < n; ++i) {
    x[i] = (float)std::exp((double)(x[i] - mx));
    sum = sum + x[i];
  }
  if (sum == 0 || std::isnan(sum) || std::isinf(sum)) return 1;
  float inv = 1 / sum;
  for (int i = 0; i < n; ++i) x[i] = x[i] * inv;
  return 0;
}

// simd.VecSiLUMul (vec_dispatch_asm.go:96-103 → kernels/activation.go:15-24):
// s = x / (1 + float32(exp(float64(-x)))), then s*up.
ORC_API void orc_silu_mul(float* dst, const float* a, const float* b, int n) {
  for (int i = 0; i < n; ++i) {
    float xv = a[i];
    float s = xv / (1.0f + (float)std::exp((double)(-xv)));
    dst[i] = s * b[i];
  }
}

// Routing of moeForwardWithREAP (model/moe.go:220-280): softmax over all
// experts, top-k by repeated strict '>' argmax starting from -1 (ties and the
// scan order give the lowest id), optional renormalisation by the selected sum.
// Writes ids/weights (length top_k); returns how many were selected.
ORC_API int orc_moe_route(const float* logits, int num_experts, int top_k, int norm_topk,
                          int* ids, float* weights) {
  if (num_experts <= 0) return 0;
  if (top_k <= 0) top_k = 8;
  if (top_k > num_experts) top_k = num_experts;
  std::vector<float> p(logits, logits + num_experts);
  if (orc_softmax(p.data(), num_experts)) return -1;
  int n = 0;
  for (int i = 0; i < top_k; ++i) {
    int best = -1;
    float bs = -1.f;
    for (int j = 0; j < num_experts; ++j) {
      if (p[j] > bs) {
        bool picked = false;
        for (int k = 0; k < n; ++k) picked |= ids[k] == j;
        if (!picked) {
          best = j;
          bs = p[j];
        }
      }
    }
    if (best >= 0) {
      ids[n] = best;
      weights[n] = bs;
      ++n;
    }
  }
  if (norm_topk && n > 0) {
    float sum = 0.f;
    for (int k = 0; k < n; ++k) sum = sum + weights[k];
    if (sum > 0)
      for (int k = 0; k < n; ++k) weights[k] = weights[k] / sum;
  }
  return n;
}

// The expert part of moeForwardWithREAP (model/moe.go:282-344) for MLX 4-bit
// experts stored back to back: gate/up [E][inter,hidden], down [E][hidden,inter]
// (all with group size gs).  For each selected expert in selection order:
// Gemv2To(gate, up) → SiLU·mul → GemvTo(down); out += weight*down, experts
// accumulated in selection order.
ORC_API int orc_moe_experts(float* out, const float* x, int hidden, int inter, int gs,
                            const uint32_t* gate_w, const float* gate_s, const float* gate_b,
                            const uint32_t* up_w, const float* up_s, const float* up_b,
                            const uint32_t* down_w, const float* down_s, const float* down_b,
                            const int* ids, const float* weights, int n_sel) {
  if (hidden <= 0 || inter <= 0 || gs <= 0 || hidden % gs || inter % gs) return 1;
  size_t gu_w = (size_t)inter * (hidden / 8), gu_s = (size_t)inter * (hidden / gs);
  size_t dn_w = (size_t)hidden * (inter / 8), dn_s = (size_t)hidden * (inter / gs);
  std::vector<float> gate(inter), up(inter), down(hidden);
  for (int i = 0; i < hidden; ++i) out[i] = 0.f;
  for (int k = 0; k < n_sel; ++k) {
    size_t e = (size_t)ids[k];
    mlx_gemv_impl(gate.data(), x, gate_w + e * gu_w, gate_s + e * gu_s, gate_b + e * gu_s,
                  inter, hidden, gs, 4, 1);
    mlx_gemv_impl(up.data(), x, up_w + e * gu_w, up_s + e * gu_s, up_b + e * gu_s, inter,
                  hidden, gs, 4, 1);
    orc_silu_mul(gate.data(), gate.data(), up.data(), inter);
    mlx_gemv_impl(down.data(), gate.data(), down_w + e * dn_w, down_s + e * dn_s,
                  down_b + e * dn_s, hidden, inter, gs, 4, 1);
    for (int i = 0; i < hidden; ++i) out[i] = out[i] + weights[k] * down[i];
  }
  return 0;
}
