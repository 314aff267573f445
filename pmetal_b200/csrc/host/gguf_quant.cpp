// Host-side GGUF block quantisers and dequantisers (C++17, multi-threaded over blocks).
//
// Formats are the ggml block layouts; the quantisation routines reproduce, bit for bit, the behaviour of the
// reference's pure-CPU quantisers (crates/pmetal-gguf/src/quantize.rs:89-330,583-856 and
// crates/pmetal-gguf/src/k_quants.rs:815-1323): round-half-away-from-zero everywhere, signed-absmax scales for
// Q4_0/Q5_0, iterative scale/min refinement for the K-quants, K-quant blocks shorter than 256 elements left
// all-zero, 32-element formats zero-padded.
//
// C ABI (all sizes in elements; buffers are caller-owned):
//   int      pm_gguf_block_elems(int type)          elements per block, 0 if the type is unknown
//   int      pm_gguf_block_bytes(int type)          bytes per block
//   int64_t  pm_gguf_row_bytes(int type, int64_t n) bytes needed for n elements (whole blocks)
//   int      pm_gguf_quantize(int type, const float* src, void* dst, int64_t n, int threads)
//   int      pm_gguf_dequantize(int type, const void* src, float* dst, int64_t n, int threads)
// Return codes: 0 ok, -1 unknown type, -2 quantisation not available for the type (dequantise-only).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

// ---------------------------------------------------------------------------------------- scalar helpers
inline int rnd(float v) { return static_cast<int>(std::lround(v)); }   // half away from zero
inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

inline uint16_t f32_to_f16(float f) {          // round to nearest even, IEEE binary16
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t mant = x & 0x007fffffu;
  const int exp = static_cast<int>((x >> 23) & 0xff);
  if (exp == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (mant ? (0x0200u | (mant >> 13)) : 0));
  const int e = exp - 127 + 15;
  if (e >= 0x1f) return static_cast<uint16_t>(sign | 0x7c00u);
  if (e <= 0) {
    if (e < -10) return static_cast<uint16_t>(sign);
    const uint32_t m = mant | 0x00800000u;
    const int shift = 14 - e;
    uint32_t half = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(e) << 10) | (mant >> 13);
  const uint32_t rem = mant & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, mant = h & 0x3ffu, out;
  if (exp == 0) {
    if (mant == 0) {
      out = sign;
    } else {
      int e = -1;
      do { ++e; mant <<= 1; } while (!(mant & 0x400u));
      out = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((mant & 0x3ffu) << 13);
    }
  } else if (exp == 0x1f) {
    out = sign | 0x7f800000u | (mant << 13);
  } else {
    out = sign | ((exp + 112) << 23) | (mant << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

inline void put16(uint8_t* p, uint16_t v) { p[0] = static_cast<uint8_t>(v); p[1] = static_cast<uint8_t>(v >> 8); }
inline uint16_t get16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
inline void put32(uint8_t* p, uint32_t v) { for (int i = 0; i < 4; ++i) p[i] = static_cast<uint8_t>(v >> (8 * i)); }
inline uint32_t get32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | (static_cast<uint32_t>(p[3]) << 24); }

// value with the largest finite magnitude (sign kept); `finite_only` mirrors the two reference variants
inline float signed_absmax(const float* x, int n, bool finite_only) {
  float best = 0.f, amax = 0.f;
  for (int i = 0; i < n; ++i) {
    if (finite_only && !std::isfinite(x[i])) continue;
    const float a = std::fabs(x[i]);
    if (a > amax) { amax = a; best = x[i]; }
  }
  return best;
}

inline void finite_min_max(const float* x, int n, float* mn, float* mx) {
  float lo = INFINITY, hi = -INFINITY;
  for (int i = 0; i < n; ++i)
    if (std::isfinite(x[i])) { lo = std::min(lo, x[i]); hi = std::max(hi, x[i]); }
  if (n == 0 || !std::isfinite(lo) || !std::isfinite(hi)) { lo = 0.f; hi = 0.f; }
  *mn = lo; *mx = hi;
}

// ggml type ids
enum : int {
  T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q8_1 = 9,
  T_Q2K = 10, T_Q3K = 11, T_Q4K = 12, T_Q5K = 13, T_Q6K = 14, T_Q8K = 15, T_IQ4_NL = 20, T_IQ4_XS = 23,
  T_BF16 = 30, T_TQ1_0 = 34, T_TQ2_0 = 35, T_MXFP4 = 39, T_NVFP4 = 40, T_Q1_0 = 41,
};

struct Fmt { int type, elems, bytes; };
constexpr Fmt kFormats[] = {
    {T_F32, 1, 4},     {T_F16, 1, 2},     {T_BF16, 1, 2},    {T_Q4_0, 32, 18},  {T_Q4_1, 32, 20},  {T_Q5_0, 32, 22},
    {T_Q5_1, 32, 24},  {T_Q8_0, 32, 34},  {T_Q8_1, 32, 36},  {T_Q2K, 256, 84},  {T_Q3K, 256, 110}, {T_Q4K, 256, 144},
    {T_Q5K, 256, 176}, {T_Q6K, 256, 210}, {T_Q8K, 256, 292}, {T_IQ4_NL, 32, 18}, {T_IQ4_XS, 256, 136}, {T_MXFP4, 32, 17},
    {T_TQ1_0, 256, 54}, {T_TQ2_0, 256, 66}, {T_NVFP4, 64, 36},  {T_Q1_0, 128, 18},
};
const Fmt* find_fmt(int type) {
  for (const Fmt& f : kFormats)
    if (f.type == type) return &f;
  return nullptr;
}

// ---------------------------------------------------------------------------------------- 32-element formats
// `n` is the number of valid elements in the block (< 32 only for the last block; the rest reads as zero).
void enc_q4_0(const float* x, int n, uint8_t* o) {
  const float d = signed_absmax(x, n, false) / -8.f;
  const float id = d == 0.f ? 0.f : 1.f / d;
  put16(o, f32_to_f16(d));
  for (int i = 0; i < 16; ++i) {
    const float a = i < n ? x[i] : 0.f, b = i + 16 < n ? x[i + 16] : 0.f;
    o[2 + i] = static_cast<uint8_t>(clampi(rnd(a * id + 8.5f), 0, 15) | (clampi(rnd(b * id + 8.5f), 0, 15) << 4));
  }
}
void enc_q4_1(const float* x, int n, uint8_t* o) {
  float mn, mx;
  finite_min_max(x, n, &mn, &mx);
  const float d = (mx - mn) / 15.f, id = d == 0.f ? 0.f : 1.f / d;
  put16(o, f32_to_f16(d));
  put16(o + 2, f32_to_f16(mn));
  for (int i = 0; i < 16; ++i) {
    const float a = i < n ? x[i] : 0.f, b = i + 16 < n ? x[i + 16] : 0.f;
    o[4 + i] = static_cast<uint8_t>(clampi(rnd((a - mn) * id), 0, 15) | (clampi(rnd((b - mn) * id), 0, 15) << 4));
  }
}
void enc_q5(const float* x, int n, uint8_t* o, bool with_min) {
  float d, mn = 0.f, id;
  if (with_min) {
    float mx;
    finite_min_max(x, n, &mn, &mx);
    d = (mx - mn) / 31.f;
  } else {
    d = signed_absmax(x, n, true) / -16.f;
  }
  id = d == 0.f ? 0.f : 1.f / d;
  uint32_t qh = 0;
  uint8_t* qs = o + (with_min ? 8 : 6);
  for (int i = 0; i < 16; ++i) {
    const float a = i < n ? x[i] : 0.f, b = i + 16 < n ? x[i + 16] : 0.f;
    const int q0 = with_min ? clampi(rnd((a - mn) * id), 0, 31) : clampi(rnd(a * id + 16.5f), 0, 31);
    const int q1 = with_min ? clampi(rnd((b - mn) * id), 0, 31) : clampi(rnd(b * id + 16.5f), 0, 31);
    qs[i] = static_cast<uint8_t>((q0 & 15) | ((q1 & 15) << 4));
    qh |= static_cast<uint32_t>(q0 >> 4) << i;
    qh |= static_cast<uint32_t>(q1 >> 4) << (i + 16);
  }
  put16(o, f32_to_f16(d));
  if (with_min) put16(o + 2, f32_to_f16(mn));
  put32(o + (with_min ? 4 : 2), qh);
}
void enc_q5_0(const float* x, int n, uint8_t* o) { enc_q5(x, n, o, false); }
void enc_q5_1(const float* x, int n, uint8_t* o) { enc_q5(x, n, o, true); }
void enc_q8(const float* x, int n, uint8_t* o, bool with_sum) {
  float amax = 0.f;
  for (int i = 0; i < n; ++i) amax = std::max(amax, std::fabs(x[i]));
  const float d = amax / 127.f, id = amax == 0.f ? 0.f : 127.f / amax;
  int sum = 0;
  uint8_t* qs = o + (with_sum ? 4 : 2);
  for (int i = 0; i < 32; ++i) {
    const int q = i < n ? clampi(rnd(x[i] * id), -127, 127) : 0;
    qs[i] = static_cast<uint8_t>(static_cast<int8_t>(q));
    sum += q;
  }
  put16(o, f32_to_f16(d));
  if (with_sum) put16(o + 2, f32_to_f16(static_cast<float>(sum) * d));
}
void enc_q8_0(const float* x, int n, uint8_t* o) { enc_q8(x, n, o, false); }
void enc_q8_1(const float* x, int n, uint8_t* o) { enc_q8(x, n, o, true); }

void dec_q4_0(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b));
  for (int i = 0; i < 16; ++i) {
    y[i] = d * ((b[2 + i] & 15) - 8);
    y[i + 16] = d * ((b[2 + i] >> 4) - 8);
  }
}
void dec_q4_1(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b)), m = f16_to_f32(get16(b + 2));
  for (int i = 0; i < 16; ++i) {
    y[i] = d * (b[4 + i] & 15) + m;
    y[i + 16] = d * (b[4 + i] >> 4) + m;
  }
}
void dec_q5_0(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b));
  const uint32_t qh = get32(b + 2);
  for (int i = 0; i < 16; ++i) {
    const int q0 = (b[6 + i] & 15) | (((qh >> i) & 1) << 4), q1 = (b[6 + i] >> 4) | (((qh >> (i + 16)) & 1) << 4);
    y[i] = d * (q0 - 16);
    y[i + 16] = d * (q1 - 16);
  }
}
void dec_q5_1(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b)), m = f16_to_f32(get16(b + 2));
  const uint32_t qh = get32(b + 4);
  for (int i = 0; i < 16; ++i) {
    const int q0 = (b[8 + i] & 15) | (((qh >> i) & 1) << 4), q1 = (b[8 + i] >> 4) | (((qh >> (i + 16)) & 1) << 4);
    y[i] = d * q0 + m;
    y[i + 16] = d * q1 + m;
  }
}
void dec_q8_0(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b));
  for (int i = 0; i < 32; ++i) y[i] = d * static_cast<int8_t>(b[2 + i]);
}
void dec_q8_1(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b));
  for (int i = 0; i < 32; ++i) y[i] = d * static_cast<int8_t>(b[4 + i]);
}

constexpr int8_t kIq4Values[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
void dec_iq4_nl(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b));
  for (int i = 0; i < 16; ++i) {
    y[i] = d * kIq4Values[b[2 + i] & 15];
    y[i + 16] = d * kIq4Values[b[2 + i] >> 4];
  }
}
// MXFP4: one E8M0 scale byte, then 16 bytes of E2M1 codes (element i low nibble, i+16 high nibble)
constexpr float kE2M1[16] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, -0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f};
inline float e8m0_half(uint8_t e) {   // 2^(e-127) / 2, with the subnormal cases of an all-zero exponent
  uint32_t bits = e < 2 ? (0x00200000u << e) : (static_cast<uint32_t>(e - 1) << 23);
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}
void dec_mxfp4(const uint8_t* b, float* y) {
  const float d = e8m0_half(b[0]);
  for (int i = 0; i < 16; ++i) {
    y[i] = d * kE2M1[b[1 + i] & 15];
    y[i + 16] = d * kE2M1[b[1 + i] >> 4];
  }
}
void enc_mxfp4(const float* x, int n, uint8_t* o) {
  float amax = 0.f;
  for (int i = 0; i < n; ++i)
    if (std::isfinite(x[i])) amax = std::max(amax, std::fabs(x[i]));
  const int e = amax > 0.f ? clampi(static_cast<int>(std::floor(std::log2(amax))) - 2 + 127, 0, 255) : 0;
  o[0] = static_cast<uint8_t>(e);
  const float d = e8m0_half(static_cast<uint8_t>(e));
  auto code = [&](float v) {
    int best = 0;
    float err = INFINITY;
    for (int c = 0; c < 16; ++c) {
      const float e2 = std::fabs(kE2M1[c] * d - v);
      if (e2 < err) { err = e2; best = c; }
    }
    return best;
  };
  for (int i = 0; i < 16; ++i) {
    const float a = i < n ? x[i] : 0.f, b = i + 16 < n ? x[i + 16] : 0.f;
    o[1 + i] = static_cast<uint8_t>(code(a) | (code(b) << 4));
  }
}

// ---------------------------------------------------------------------------------------- NVFP4 / ternary / 1-bit
// UE4M3 scale byte (unsigned E4M3 with an extra factor 1/2 on decode), as the reference's fp4.rs defines it.
inline float ue4m3_to_f32(uint8_t x) {
  if (x == 0 || x == 0x7f) return 0.f;
  const int e = (x >> 3) & 15, m = x & 7;
  const float raw = e == 0 ? static_cast<float>(m) * std::ldexp(1.f, -9) : (1.f + static_cast<float>(m) / 8.f) * std::ldexp(1.f, e - 7);
  return raw * 0.5f;
}
inline uint8_t f32_to_ue4m3(float x) {
  if (!(x > 0.f) || !std::isfinite(x)) return 0;
  if (x > 448.f) x = 448.f;
  uint32_t bits;
  std::memcpy(&bits, &x, 4);
  const int fe = static_cast<int>((bits >> 23) & 0xff) - 127, fm = static_cast<int>((bits >> 20) & 7);
  int e = fe + 7;
  if (e <= 0) {
    const int man = static_cast<int>(x * 512.f + 0.5f);
    return static_cast<uint8_t>(man > 7 ? 7 : (man < 1 ? 0 : man));
  }
  if (e >= 15) return 0x7e;
  int m = fm + static_cast<int>((bits >> 19) & 1);
  if (m > 7) {
    m = 0;
    if (++e >= 15) return 0x7e;
  }
  return static_cast<uint8_t>((e << 3) | m);
}
inline int nearest_e2m1(float v, float d) {
  int best = 0;
  float err = std::fabs(kE2M1[0] * d - v);
  for (int c = 1; c < 16; ++c) {
    const float e2 = std::fabs(kE2M1[c] * d - v);
    if (e2 < err) { err = e2; best = c; }
  }
  return best;
}
// NVFP4: 64 elements = 4 sub-blocks of 16; bytes 0-3 scales, then 4 x 8 nibble bytes (element i low, i + 8 high)
void enc_nvfp4(const float* x, int n, uint8_t* o) {
  std::memset(o, 0, 36);
  for (int sub = 0; sub < 4; ++sub) {
    const int s0 = sub * 16;
    float amax = 0.f;
    for (int i = s0; i < std::min(s0 + 16, n); ++i)
      if (std::isfinite(x[i])) amax = std::max(amax, std::fabs(x[i]));
    const uint8_t sb = f32_to_ue4m3(amax / 6.f);
    const float d = ue4m3_to_f32(sb);
    o[sub] = sb;
    for (int i = 0; i < 8; ++i) {
      const float a = s0 + i < n ? x[s0 + i] : 0.f, b = s0 + i + 8 < n ? x[s0 + i + 8] : 0.f;
      o[4 + sub * 8 + i] = static_cast<uint8_t>(nearest_e2m1(a, d) | (nearest_e2m1(b, d) << 4));
    }
  }
}
void dec_nvfp4(const uint8_t* b, float* y) {
  for (int sub = 0; sub < 4; ++sub) {
    const float d = ue4m3_to_f32(b[sub]);
    for (int i = 0; i < 8; ++i) {
      y[sub * 16 + i] = d * kE2M1[b[4 + sub * 8 + i] & 15];
      y[sub * 16 + i + 8] = d * kE2M1[b[4 + sub * 8 + i] >> 4];
    }
  }
}
inline int trit(float v, float inv) {
  float q = std::round(v * inv);
  q = q < -1.f ? -1.f : (q > 1.f ? 1.f : q);
  return static_cast<int>(q) + 1;
}
inline float finite_amax(const float* x, int n) {
  float amax = 0.f;
  for (int i = 0; i < n; ++i)
    if (std::isfinite(x[i])) amax = std::max(amax, std::fabs(x[i]));
  return amax;
}
// TQ1_0 {qs[48], qh[4], d}: five trits per byte stored as ceil(q * 256 / 243); strides 32, then 16, then 4
void enc_tq1_0(const float* x, int n, uint8_t* o) {
  const float amax = finite_amax(x, n), inv = amax > 0.f ? 1.f / amax : 0.f;
  auto at = [&](int i) { return i < n ? x[i] : 0.f; };
  int base = 0;
  for (int m = 0; m < 32; ++m) {
    int q = 0;
    for (int k = 0; k < 5; ++k) q = q * 3 + trit(at(base + m + k * 32), inv);
    o[m] = static_cast<uint8_t>((q * 256 + 242) / 243);
  }
  base += 160;
  for (int m = 0; m < 16; ++m) {
    int q = 0;
    for (int k = 0; k < 5; ++k) q = q * 3 + trit(at(base + m + k * 16), inv);
    o[32 + m] = static_cast<uint8_t>((q * 256 + 242) / 243);
  }
  base += 80;
  for (int j = 0; j < 4; ++j) {
    int q = 0;
    for (int m = 0; m < 4; ++m) q = q * 3 + trit(at(base + j + m * 4), inv);
    q = std::min(q * 3, 255);
    o[48 + j] = static_cast<uint8_t>((q * 256 + 242) / 243);
  }
  put16(o + 52, f32_to_f16(amax));
}
inline int trit_of(uint8_t packed, int k) {     // k-th most significant of five trits
  static const int pow3[5] = {1, 3, 9, 27, 81};
  const uint16_t q = static_cast<uint16_t>(packed * pow3[k]);      // shifts the wanted trit to the top
  return ((q & 0xff) * 3) >> 8;
}
void dec_tq1_0(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b + 52));
  int base = 0;
  for (int k = 0; k < 5; ++k)
    for (int m = 0; m < 32; ++m) y[base + k * 32 + m] = d * static_cast<float>(trit_of(b[m], k) - 1);
  base += 160;
  for (int k = 0; k < 5; ++k)
    for (int m = 0; m < 16; ++m) y[base + k * 16 + m] = d * static_cast<float>(trit_of(b[32 + m], k) - 1);
  base += 80;
  for (int m = 0; m < 4; ++m)
    for (int j = 0; j < 4; ++j) y[base + m * 4 + j] = d * static_cast<float>(trit_of(b[48 + j], m) - 1);
}
// TQ2_0 {qs[64], d}: two bits per trit, four elements 32 apart per byte
void enc_tq2_0(const float* x, int n, uint8_t* o) {
  const float amax = finite_amax(x, n), inv = amax > 0.f ? 1.f / amax : 0.f;
  for (int h = 0; h < 2; ++h)
    for (int m = 0; m < 32; ++m) {
      int q = 0;
      for (int k = 0; k < 4; ++k) {
        const int i = h * 128 + m + k * 32;
        q |= (trit(i < n ? x[i] : 0.f, inv) & 3) << (2 * k);
      }
      o[h * 32 + m] = static_cast<uint8_t>(q);
    }
  put16(o + 64, f32_to_f16(amax));
}
void dec_tq2_0(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b + 64));
  for (int h = 0; h < 2; ++h)
    for (int k = 0; k < 4; ++k)
      for (int m = 0; m < 32; ++m) y[h * 128 + k * 32 + m] = d * static_cast<float>(((b[h * 32 + m] >> (2 * k)) & 3) - 1);
}
// Q1_0 {d f16 = mean |x| over 128, 16 bytes of sign bits (bit set = non-negative)}
void enc_q1_0(const float* x, int n, uint8_t* o) {
  float sum = 0.f;
  for (int i = 0; i < n; ++i)
    if (std::isfinite(x[i])) sum += std::fabs(x[i]);
  put16(o, f32_to_f16(sum / 128.f));
  std::memset(o + 2, 0, 16);
  for (int i = 0; i < 128; ++i)
    if ((i < n ? x[i] : 0.f) >= 0.f) o[2 + i / 8] |= static_cast<uint8_t>(1u << (i % 8));
}
void dec_q1_0(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b));
  for (int i = 0; i < 128; ++i) y[i] = ((b[2 + i / 8] >> (i % 8)) & 1) ? d : -d;
}

// ---------------------------------------------------------------------------------------- K-quant helpers
// Scale and (negated) minimum for an asymmetric sub-block: x ~ scale * q - min_neg, q in [0, nmax].
void fit_scale_min(int nmax, int ntry, const float* x, int n, float* scale_out, float* min_neg_out) {
  uint8_t q[32] = {0};
  float lo = x[0], hi = x[0];
  for (int i = 1; i < n; ++i) { lo = std::min(lo, x[i]); hi = std::max(hi, x[i]); }
  if (hi == lo) { *scale_out = 0.f; *min_neg_out = 0.f; return; }
  float mn = std::min(lo, 0.f);
  float inv = static_cast<float>(nmax) / (hi - mn);
  float scale = 1.f / inv;
  for (int it = 0; it < ntry; ++it) {
    float sum_lx = 0.f;
    int sum_l2 = 0;
    bool changed = false;
    for (int i = 0; i < n; ++i) {
      const int li = clampi(rnd(inv * (x[i] - mn)), 0, nmax);
      if (static_cast<uint8_t>(li) != q[i]) { q[i] = static_cast<uint8_t>(li); changed = true; }
      sum_lx += (x[i] - mn) * static_cast<float>(li);
      sum_l2 += li * li;
    }
    if (sum_l2 == 0) break;
    scale = sum_lx / static_cast<float>(sum_l2);
    float resid = 0.f;
    for (int i = 0; i < n; ++i) resid += x[i] - scale * static_cast<float>(q[i]);
    mn = std::min(resid / static_cast<float>(n), 0.f);
    inv = 1.f / scale;
    if (!changed) break;
  }
  *scale_out = scale;
  *min_neg_out = -mn;
}

// One coordinate-descent sweep shared by the symmetric fitters: try to move each level to the value that is
// optimal given the others, keep the move if it raises (sum w x l)^2 / (sum w l^2). Returns moves made.
int refine_levels(const float* x, int n, int nmax, int8_t* lv, int bias, float* sum_lx, float* sum_l2) {
  int moved = 0;
  for (int i = 0; i < n; ++i) {
    const float w = x[i] * x[i];
    const int l = lv[i] - bias;
    float slx = *sum_lx - w * x[i] * static_cast<float>(l);
    if (slx > 0.f) {
      float sl2 = *sum_l2 - w * static_cast<float>(l * l);
      const int nl = clampi(rnd(x[i] * sl2 / slx), -nmax, nmax - 1);
      if (nl != l) {
        slx += w * x[i] * static_cast<float>(nl);
        sl2 += w * static_cast<float>(nl * nl);
        if (sl2 > 0.f && slx * slx * *sum_l2 > *sum_lx * *sum_lx * sl2) {
          lv[i] = static_cast<int8_t>(nl + bias);
          *sum_lx = slx;
          *sum_l2 = sl2;
          ++moved;
        }
      }
    }
  }
  return moved;
}

// Symmetric sub-block fit used by Q6_K: levels in [-nmax, nmax-1] stored with +nmax bias, weights x^2.
float fit_symmetric_q6(const float* x, int n, int nmax, int8_t* lv) {
  std::fill(lv, lv + n, 0);
  const float mx = signed_absmax(x, n, false);
  if (mx == 0.f) return 0.f;
  float inv = -static_cast<float>(nmax) / mx;
  float sum_lx = 0.f, sum_l2 = 0.f;
  for (int i = 0; i < n; ++i) {
    const int l = clampi(rnd(inv * x[i]), -nmax, nmax - 1);
    lv[i] = static_cast<int8_t>(l + nmax);
    const float w = x[i] * x[i];
    sum_lx += w * x[i] * static_cast<float>(l);
    sum_l2 += w * static_cast<float>(l * l);
  }
  float scale = sum_lx / sum_l2;
  float best = scale * sum_lx;
  for (int it = 0; it < 3; ++it) {
    inv = 1.f / scale;
    float slx = 0.f, sl2 = 0.f;
    bool changed = false;
    for (int i = 0; i < n; ++i) {
      const int l = clampi(rnd(inv * x[i]), -nmax, nmax - 1);
      if (l + nmax != lv[i]) changed = true;
      const float w = x[i] * x[i];
      slx += w * x[i] * static_cast<float>(l);
      sl2 += w * static_cast<float>(l * l);
    }
    if (!changed || sl2 == 0.f || slx * slx <= best * sl2) break;
    for (int i = 0; i < n; ++i) lv[i] = static_cast<int8_t>(nmax + clampi(rnd(inv * x[i]), -nmax, nmax - 1));
    sum_lx = slx;
    sum_l2 = sl2;
    scale = sum_lx / sum_l2;
    best = scale * sum_lx;
  }
  for (int it = 0; it < 5; ++it) {
    if (refine_levels(x, n, nmax, lv, nmax, &sum_lx, &sum_l2) == 0) break;
    scale = sum_lx / sum_l2;
  }
  return scale;
}

// Symmetric sub-block fit used by Q3_K (levels in [-nmax, nmax-1], weights x^2, no re-scale passes).
float fit_symmetric_q3(const float* x, int n, int nmax) {
  int8_t lv[16];
  const float mx = signed_absmax(x, n, false);
  if (mx == 0.f) return 0.f;
  const float inv = -static_cast<float>(nmax) / mx;
  float sum_lx = 0.f, sum_l2 = 0.f;
  for (int i = 0; i < n; ++i) {
    const int l = clampi(rnd(inv * x[i]), -nmax, nmax - 1);
    lv[i] = static_cast<int8_t>(l);
    const float w = x[i] * x[i];
    sum_lx += w * x[i] * static_cast<float>(l);
    sum_l2 += w * static_cast<float>(l * l);
  }
  for (int it = 0; it < 5; ++it)
    if (refine_levels(x, n, nmax, lv, 0, &sum_lx, &sum_l2) == 0) break;
  return sum_lx / sum_l2;
}

// 6-bit (scale, min) pair j of the 12-byte Q4_K/Q5_K scale field
inline void unpack_scale_min(int j, const uint8_t* q, int* sc, int* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (q[j + 4] & 15) | ((q[j - 4] >> 6) << 4);
    *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// Shared front half of Q4_K / Q5_K: per-32 fits, 6-bit packing, d/dmin, then levels against the decoded scales.
void q45k_levels(const float* x, int nmax, uint8_t* d_out, uint8_t* scales12, uint8_t* lv) {
  float sc[8], mn[8], max_sc = 0.f, max_mn = 0.f;
  for (int j = 0; j < 8; ++j) {
    fit_scale_min(nmax, 5, x + 32 * j, 32, &sc[j], &mn[j]);
    max_sc = std::max(max_sc, sc[j]);
    max_mn = std::max(max_mn, mn[j]);
  }
  const float inv_sc = max_sc > 0.f ? 63.f / max_sc : 0.f, inv_mn = max_mn > 0.f ? 63.f / max_mn : 0.f;
  std::memset(scales12, 0, 12);
  for (int j = 0; j < 8; ++j) {
    const uint8_t ls = static_cast<uint8_t>(std::min(rnd(inv_sc * sc[j]), 63));
    const uint8_t lm = static_cast<uint8_t>(std::min(rnd(inv_mn * mn[j]), 63));
    if (j < 4) {
      scales12[j] = ls;
      scales12[j + 4] = lm;
    } else {
      scales12[j + 4] = static_cast<uint8_t>((ls & 15) | ((lm & 15) << 4));
      scales12[j - 4] |= static_cast<uint8_t>((ls >> 4) << 6);
      scales12[j] |= static_cast<uint8_t>((lm >> 4) << 6);
    }
  }
  const uint16_t dh = f32_to_f16(max_sc / 63.f), mh = f32_to_f16(max_mn / 63.f);
  put16(d_out, dh);
  put16(d_out + 2, mh);
  const float df = f16_to_f32(dh), mf = f16_to_f32(mh);
  std::memset(lv, 0, 256);
  for (int j = 0; j < 8; ++j) {
    int s, m;
    unpack_scale_min(j, scales12, &s, &m);
    const float d = df * static_cast<float>(s);
    if (d == 0.f) continue;
    const float dm = mf * static_cast<float>(m);
    for (int i = 0; i < 32; ++i) lv[32 * j + i] = static_cast<uint8_t>(clampi(rnd((x[32 * j + i] + dm) / d), 0, nmax));
  }
}

// block layouts (bytes): Q4_K {d, dmin, scales[12], qs[128]}   Q5_K {d, dmin, scales[12], qh[32], qs[128]}
void enc_q4k(const float* x, int, uint8_t* o) {
  uint8_t lv[256];
  q45k_levels(x, 15, o, o + 4, lv);
  uint8_t* qs = o + 16;
  for (int g = 0; g < 4; ++g)
    for (int i = 0; i < 32; ++i) qs[g * 32 + i] = static_cast<uint8_t>(lv[g * 64 + i] | (lv[g * 64 + i + 32] << 4));
}
void enc_q5k(const float* x, int, uint8_t* o) {
  uint8_t lv[256];
  q45k_levels(x, 31, o, o + 4, lv);
  uint8_t *qh = o + 16, *qs = o + 48;
  std::memset(qh, 0, 32);
  for (int g = 0; g < 4; ++g)
    for (int i = 0; i < 32; ++i) {
      int a = lv[g * 64 + i], b = lv[g * 64 + i + 32];
      if (a > 15) { a -= 16; qh[i] |= static_cast<uint8_t>(1u << (2 * g)); }
      if (b > 15) { b -= 16; qh[i] |= static_cast<uint8_t>(2u << (2 * g)); }
      qs[g * 32 + i] = static_cast<uint8_t>(a | (b << 4));
    }
}
void dec_q4k(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b)), dmin = f16_to_f32(get16(b + 2));
  const uint8_t* qs = b + 16;
  for (int g = 0; g < 4; ++g) {
    int s0, m0, s1, m1;
    unpack_scale_min(2 * g, b + 4, &s0, &m0);
    unpack_scale_min(2 * g + 1, b + 4, &s1, &m1);
    for (int i = 0; i < 32; ++i) {
      y[g * 64 + i] = d * s0 * (qs[g * 32 + i] & 15) - dmin * m0;
      y[g * 64 + 32 + i] = d * s1 * (qs[g * 32 + i] >> 4) - dmin * m1;
    }
  }
}
void dec_q5k(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b)), dmin = f16_to_f32(get16(b + 2));
  const uint8_t *qh = b + 16, *qs = b + 48;
  for (int g = 0; g < 4; ++g) {
    int s0, m0, s1, m1;
    unpack_scale_min(2 * g, b + 4, &s0, &m0);
    unpack_scale_min(2 * g + 1, b + 4, &s1, &m1);
    for (int i = 0; i < 32; ++i) {
      const int a = (qs[g * 32 + i] & 15) + (((qh[i] >> (2 * g)) & 1) << 4);
      const int c = (qs[g * 32 + i] >> 4) + (((qh[i] >> (2 * g + 1)) & 1) << 4);
      y[g * 64 + i] = d * s0 * a - dmin * m0;
      y[g * 64 + 32 + i] = d * s1 * c - dmin * m1;
    }
  }
}

// Q6_K {ql[128], qh[64], scales[16] i8, d}
void enc_q6k(const float* x, int, uint8_t* o) {
  int8_t lv[256];
  float sc[16], max_sc = 0.f, max_abs = 0.f;
  for (int j = 0; j < 16; ++j) {
    sc[j] = fit_symmetric_q6(x + 16 * j, 16, 32, lv + 16 * j);
    if (std::fabs(sc[j]) > max_abs) { max_abs = std::fabs(sc[j]); max_sc = sc[j]; }
  }
  uint8_t *ql = o, *qh = o + 128;
  int8_t* scales = reinterpret_cast<int8_t*>(o + 192);
  const float inv = -128.f / max_sc;       // an all-zero block gives -inf here and NaN scales, as in the reference
  const uint16_t dh = f32_to_f16(1.f / inv);
  put16(o + 208, dh);
  const float df = f16_to_f32(dh);
  for (int j = 0; j < 16; ++j) {
    const float t = inv * sc[j];
    // NaN (0 * inf) rounds to 0 in the reference's saturating float->int cast
    scales[j] = static_cast<int8_t>(std::isnan(t) ? 0 : std::min(rnd(t), 127));
  }
  for (int j = 0; j < 16; ++j) {
    const float d = df * static_cast<float>(scales[j]);
    if (d == 0.f || std::isnan(d)) continue;
    for (int i = 0; i < 16; ++i) lv[16 * j + i] = static_cast<int8_t>(clampi(rnd(x[16 * j + i] / d), -32, 31) + 32);
  }
  for (int h = 0; h < 2; ++h)
    for (int i = 0; i < 32; ++i) {
      const int8_t* l = lv + 128 * h + i;
      ql[64 * h + i] = static_cast<uint8_t>((l[0] & 15) | ((l[64] & 15) << 4));
      ql[64 * h + i + 32] = static_cast<uint8_t>((l[32] & 15) | ((l[96] & 15) << 4));
      qh[32 * h + i] = static_cast<uint8_t>((l[0] >> 4) | ((l[32] >> 4) << 2) | ((l[64] >> 4) << 4) | ((l[96] >> 4) << 6));
    }
}
void dec_q6k(const uint8_t* b, float* y) {
  const uint8_t *ql = b, *qh = b + 128;
  const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
  const float d = f16_to_f32(get16(b + 208));
  for (int h = 0; h < 2; ++h)
    for (int i = 0; i < 32; ++i) {
      const int is = 8 * h + i / 16;
      const uint8_t hb = qh[32 * h + i];
      const int q1 = ((ql[64 * h + i] & 15) | (((hb >> 0) & 3) << 4)) - 32;
      const int q2 = ((ql[64 * h + i + 32] & 15) | (((hb >> 2) & 3) << 4)) - 32;
      const int q3 = ((ql[64 * h + i] >> 4) | (((hb >> 4) & 3) << 4)) - 32;
      const int q4 = ((ql[64 * h + i + 32] >> 4) | (((hb >> 6) & 3) << 4)) - 32;
      float* o = y + 128 * h + i;
      o[0] = d * sc[is] * q1;
      o[32] = d * sc[is + 2] * q2;
      o[64] = d * sc[is + 4] * q3;
      o[96] = d * sc[is + 6] * q4;
    }
}

// Q3_K {hmask[32], qs[64], scales[12], d}
inline int q3k_scale(const uint8_t* s, int j) {
  const int lo = j < 8 ? (s[j] & 15) : (s[j - 8] >> 4);
  return (lo | (((s[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32;
}
void enc_q3k(const float* x, int, uint8_t* o) {
  uint8_t *hmask = o, *qs = o + 32, *scales = o + 96;
  float sc[16], max_sc = 0.f;
  for (int j = 0; j < 16; ++j) {
    sc[j] = fit_symmetric_q3(x + 16 * j, 16, 4);
    if (std::fabs(sc[j]) > std::fabs(max_sc)) max_sc = sc[j];
  }
  std::memset(scales, 0, 12);
  uint16_t dh = 0;
  if (max_sc != 0.f) {
    const float inv = -32.f / max_sc;
    for (int j = 0; j < 16; ++j) {
      const int l = clampi(rnd(inv * sc[j]), -32, 31) + 32;
      if (j < 8) scales[j] = static_cast<uint8_t>(l & 15);
      else scales[j - 8] |= static_cast<uint8_t>((l & 15) << 4);
      scales[j % 4 + 8] |= static_cast<uint8_t>((l >> 4) << (2 * (j / 4)));
    }
    dh = f32_to_f16(1.f / inv);
  }
  put16(o + 108, dh);
  const float df = f16_to_f32(dh);
  int8_t lv[256] = {0};
  for (int j = 0; j < 16; ++j) {
    const float d = df * static_cast<float>(q3k_scale(scales, j));
    if (d == 0.f) continue;
    for (int i = 0; i < 16; ++i) lv[16 * j + i] = static_cast<int8_t>(clampi(rnd(x[16 * j + i] / d), -4, 3) + 4);
  }
  std::memset(hmask, 0, 32);
  for (int i = 0; i < 256; ++i)
    if (lv[i] > 3) { hmask[i & 31] |= static_cast<uint8_t>(1u << (i >> 5)); lv[i] -= 4; }
  for (int h = 0; h < 2; ++h)
    for (int i = 0; i < 32; ++i) {
      const int8_t* l = lv + 128 * h + i;
      qs[32 * h + i] = static_cast<uint8_t>(l[0] | (l[32] << 2) | (l[64] << 4) | (l[96] << 6));
    }
}
void dec_q3k(const uint8_t* b, float* y) {
  const uint8_t *hmask = b, *qs = b + 32, *scales = b + 96;
  const float d = f16_to_f32(get16(b + 108));
  for (int i = 0; i < 256; ++i) {
    const int h = i >> 7, r = i & 127, lane = r & 31, grp = r >> 5;       // grp = 2-bit slot within the byte
    const int lo = (qs[32 * h + lane] >> (2 * grp)) & 3;
    const int hi = (hmask[i & 31] >> (i >> 5)) & 1;
    y[i] = d * static_cast<float>(q3k_scale(scales, i >> 4)) * static_cast<float>(lo - (hi ? 0 : 4));
  }
}

// Q2_K {scales[16], qs[64], d, dmin}
void enc_q2k(const float* x, int, uint8_t* o) {
  uint8_t *scales = o, *qs = o + 16;
  float sc[16], mn[16], max_sc = 0.f, max_mn = 0.f;
  for (int j = 0; j < 16; ++j) {
    fit_scale_min(3, 5, x + 16 * j, 16, &sc[j], &mn[j]);
    max_sc = std::max(max_sc, sc[j]);
    max_mn = std::max(max_mn, mn[j]);
  }
  std::memset(scales, 0, 16);
  uint16_t dh = 0, mh = 0;
  if (max_sc > 0.f) {
    const float inv = 15.f / max_sc;
    for (int j = 0; j < 16; ++j) scales[j] = static_cast<uint8_t>(rnd(inv * sc[j]));
    dh = f32_to_f16(max_sc / 15.f);
  }
  if (max_mn > 0.f) {
    const float inv = 15.f / max_mn;
    for (int j = 0; j < 16; ++j) scales[j] |= static_cast<uint8_t>(static_cast<uint8_t>(rnd(inv * mn[j])) << 4);
    mh = f32_to_f16(max_mn / 15.f);
  }
  put16(o + 80, dh);
  put16(o + 82, mh);
  const float df = f16_to_f32(dh), mf = f16_to_f32(mh);
  uint8_t lv[256] = {0};
  for (int j = 0; j < 16; ++j) {
    const float d = df * static_cast<float>(scales[j] & 15);
    if (d == 0.f) continue;
    const float dm = mf * static_cast<float>(scales[j] >> 4);
    for (int i = 0; i < 16; ++i) lv[16 * j + i] = static_cast<uint8_t>(clampi(rnd((x[16 * j + i] + dm) / d), 0, 3));
  }
  for (int h = 0; h < 2; ++h)
    for (int i = 0; i < 32; ++i) {
      const uint8_t* l = lv + 128 * h + i;
      qs[32 * h + i] = static_cast<uint8_t>(l[0] | (l[32] << 2) | (l[64] << 4) | (l[96] << 6));
    }
}
void dec_q2k(const uint8_t* b, float* y) {
  const uint8_t *scales = b, *qs = b + 16;
  const float d = f16_to_f32(get16(b + 80)), dmin = f16_to_f32(get16(b + 82));
  for (int i = 0; i < 256; ++i) {
    const int h = i >> 7, r = i & 127;
    const int q = (qs[32 * h + (r & 31)] >> (2 * (r >> 5))) & 3;
    const uint8_t s = scales[i >> 4];
    y[i] = d * static_cast<float>(s & 15) * static_cast<float>(q) - dmin * static_cast<float>(s >> 4);
  }
}

// Q8_K {d f32, qs[256] i8, bsums[16] i16}
void enc_q8k(const float* x, int, uint8_t* o) {
  std::memset(o, 0, 292);
  const float mx = signed_absmax(x, 256, false);
  if (mx == 0.f) return;
  const float inv = -128.f / mx;
  int8_t* qs = reinterpret_cast<int8_t*>(o + 4);
  for (int i = 0; i < 256; ++i) qs[i] = static_cast<int8_t>(std::min(std::round(inv * x[i]), 127.f));
  for (int j = 0; j < 16; ++j) {
    int s = 0;
    for (int i = 0; i < 16; ++i) s += qs[16 * j + i];
    put16(o + 260 + 2 * j, static_cast<uint16_t>(static_cast<int16_t>(s)));
  }
  const float d = 1.f / inv;
  std::memcpy(o, &d, 4);
}
void dec_q8k(const uint8_t* b, float* y) {
  float d;
  std::memcpy(&d, b, 4);
  for (int i = 0; i < 256; ++i) y[i] = d * static_cast<int8_t>(b[4 + i]);
}

// IQ4_XS {d f16, scales_h u16, scales_l[4], qs[128]} (dequantise only)
void dec_iq4_xs(const uint8_t* b, float* y) {
  const float d = f16_to_f32(get16(b));
  const uint16_t sh = get16(b + 2);
  const uint8_t *sl = b + 4, *qs = b + 8;
  for (int j = 0; j < 8; ++j) {
    const int ls = ((sl[j / 2] >> (4 * (j % 2))) & 15) | (((sh >> (2 * j)) & 3) << 4);
    const float dl = d * static_cast<float>(ls - 32);
    for (int i = 0; i < 16; ++i) {
      y[32 * j + i] = dl * kIq4Values[qs[16 * j + i] & 15];
      y[32 * j + 16 + i] = dl * kIq4Values[qs[16 * j + i] >> 4];
    }
  }
}

using EncFn = void (*)(const float*, int, uint8_t*);
using DecFn = void (*)(const uint8_t*, float*);
EncFn encoder(int type) {
  switch (type) {
    case T_Q4_0: return enc_q4_0;  case T_Q4_1: return enc_q4_1;  case T_Q5_0: return enc_q5_0;
    case T_Q5_1: return enc_q5_1;  case T_Q8_0: return enc_q8_0;  case T_Q8_1: return enc_q8_1;
    case T_Q2K: return enc_q2k;    case T_Q3K: return enc_q3k;    case T_Q4K: return enc_q4k;
    case T_Q5K: return enc_q5k;    case T_Q6K: return enc_q6k;    case T_Q8K: return enc_q8k;
    case T_MXFP4: return enc_mxfp4;  case T_NVFP4: return enc_nvfp4;  case T_TQ1_0: return enc_tq1_0;
    case T_TQ2_0: return enc_tq2_0;  case T_Q1_0: return enc_q1_0;
    default: return nullptr;
  }
}
DecFn decoder(int type) {
  switch (type) {
    case T_Q4_0: return dec_q4_0;  case T_Q4_1: return dec_q4_1;  case T_Q5_0: return dec_q5_0;
    case T_Q5_1: return dec_q5_1;  case T_Q8_0: return dec_q8_0;  case T_Q8_1: return dec_q8_1;
    case T_Q2K: return dec_q2k;    case T_Q3K: return dec_q3k;    case T_Q4K: return dec_q4k;
    case T_Q5K: return dec_q5k;    case T_Q6K: return dec_q6k;    case T_Q8K: return dec_q8k;
    case T_IQ4_NL: return dec_iq4_nl;  case T_IQ4_XS: return dec_iq4_xs;  case T_MXFP4: return dec_mxfp4;
    case T_NVFP4: return dec_nvfp4;  case T_TQ1_0: return dec_tq1_0;  case T_TQ2_0: return dec_tq2_0;
    case T_Q1_0: return dec_q1_0;
    default: return nullptr;
  }
}

template <typename F>
void parallel_blocks(int64_t n_blocks, int threads, F&& body) {
  if (threads <= 0) threads = static_cast<int>(std::max(1u, std::thread::hardware_concurrency()));
  threads = static_cast<int>(std::min<int64_t>(threads, std::max<int64_t>(1, n_blocks / 64)));
  if (threads <= 1) { body(0, n_blocks); return; }
  std::vector<std::thread> pool;
  const int64_t per = (n_blocks + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const int64_t b0 = t * per, b1 = std::min(n_blocks, b0 + per);
    if (b0 >= b1) break;
    pool.emplace_back([&body, b0, b1] { body(b0, b1); });
  }
  for (auto& th : pool) th.join();
}

inline uint16_t f32_to_bf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((x >> 16) | 0x40);
  return static_cast<uint16_t>((x + 0x7fffu + ((x >> 16) & 1)) >> 16);
}


// ---------------------------------------------------------------------------------------------- integer dot products
// Dot product of a K-quant row with a Q8_K-quantised activation row without going through floats
// (role of crates/pmetal-gguf/src/vec_dot.rs:53-880). One routine serves every type: a block is unpacked
// into 256 integer levels, sixteen integer sub-block scales and sixteen integer sub-block minima, so that
//   x_i = d * sc[i/16] * q_i - dmin * mn[i/16],   y_i = yd * yq_i
//   dot = yd * ( d * sum_j sc_j * sum_{i in j} q_i yq_i  -  dmin * sum_j mn_j * bsum_j )
// with all inner sums exact in int32 (|q| <= 128, |yq| <= 128, 16 terms, |sc| <= 255).
struct Levels {
  int8_t q[256];
  int sc[16];
  int mn[16];
  float d, dmin;
};

bool unpack_levels(int type, const uint8_t* b, Levels* L) {
  for (int j = 0; j < 16; ++j) L->mn[j] = 0;
  L->dmin = 0.f;
  switch (type) {
    case T_Q2K: {
      const uint8_t *scales = b, *qs = b + 16;
      L->d = f16_to_f32(get16(b + 80));
      L->dmin = f16_to_f32(get16(b + 82));
      for (int j = 0; j < 16; ++j) { L->sc[j] = scales[j] & 15; L->mn[j] = scales[j] >> 4; }
      for (int i = 0; i < 256; ++i) {
        const int h = i >> 7, r = i & 127;
        L->q[i] = static_cast<int8_t>((qs[32 * h + (r & 31)] >> (2 * (r >> 5))) & 3);
      }
      return true;
    }
    case T_Q3K: {
      const uint8_t *hmask = b, *qs = b + 32, *scales = b + 96;
      L->d = f16_to_f32(get16(b + 108));
      for (int j = 0; j < 16; ++j) L->sc[j] = q3k_scale(scales, j);
      for (int i = 0; i < 256; ++i) {
        const int h = i >> 7, r = i & 127;
        const int lo = (qs[32 * h + (r & 31)] >> (2 * (r >> 5))) & 3;
        const int hi = (hmask[i & 31] >> (i >> 5)) & 1;
        L->q[i] = static_cast<int8_t>(lo - (hi ? 0 : 4));
      }
      return true;
    }
    case T_Q4K:
    case T_Q5K: {
      L->d = f16_to_f32(get16(b));
      L->dmin = f16_to_f32(get16(b + 2));
      const uint8_t* qh = b + 16;
      const uint8_t* qs = type == T_Q4K ? b + 16 : b + 48;
      for (int j = 0; j < 8; ++j) {
        int sv, mv;
        unpack_scale_min(j, b + 4, &sv, &mv);
        L->sc[2 * j] = L->sc[2 * j + 1] = sv;
        L->mn[2 * j] = L->mn[2 * j + 1] = mv;
      }
      for (int g = 0; g < 4; ++g)
        for (int i = 0; i < 32; ++i) {
          int lo = qs[g * 32 + i] & 15, hi = qs[g * 32 + i] >> 4;
          if (type == T_Q5K) {
            lo += ((qh[i] >> (2 * g)) & 1) << 4;
            hi += ((qh[i] >> (2 * g + 1)) & 1) << 4;
          }
          L->q[g * 64 + i] = static_cast<int8_t>(lo);
          L->q[g * 64 + 32 + i] = static_cast<int8_t>(hi);
        }
      return true;
    }
    case T_Q6K: {
      const uint8_t *ql = b, *qh = b + 128;
      const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
      L->d = f16_to_f32(get16(b + 208));
      for (int j = 0; j < 16; ++j) L->sc[j] = sc[j];
      for (int h = 0; h < 2; ++h)
        for (int i = 0; i < 32; ++i) {
          const uint8_t hb = qh[32 * h + i];
          int8_t* o = L->q + 128 * h + i;
          o[0] = static_cast<int8_t>(((ql[64 * h + i] & 15) | (((hb >> 0) & 3) << 4)) - 32);
          o[32] = static_cast<int8_t>(((ql[64 * h + i + 32] & 15) | (((hb >> 2) & 3) << 4)) - 32);
          o[64] = static_cast<int8_t>(((ql[64 * h + i] >> 4) | (((hb >> 4) & 3) << 4)) - 32);
          o[96] = static_cast<int8_t>(((ql[64 * h + i + 32] >> 4) | (((hb >> 6) & 3) << 4)) - 32);
        }
      return true;
    }
    case T_Q8K: {
      std::memcpy(&L->d, b, 4);
      for (int j = 0; j < 16; ++j) L->sc[j] = 1;
      std::memcpy(L->q, b + 4, 256);
      return true;
    }
    default:
      return false;
  }
}

// one 256-element block of `type` against one Q8_K block
inline float block_dot_q8k(const Levels& L, const uint8_t* yb) {
  float yd;
  std::memcpy(&yd, yb, 4);
  const int8_t* yq = reinterpret_cast<const int8_t*>(yb + 4);
  int64_t acc = 0, macc = 0;
  for (int j = 0; j < 16; ++j) {
    int s = 0;
    for (int i = 0; i < 16; ++i) s += static_cast<int>(L.q[16 * j + i]) * static_cast<int>(yq[16 * j + i]);
    acc += static_cast<int64_t>(L.sc[j]) * s;
    macc += static_cast<int64_t>(L.mn[j]) * static_cast<int16_t>(get16(yb + 260 + 2 * j));
  }
  return yd * (L.d * static_cast<float>(acc) - L.dmin * static_cast<float>(macc));
}

double row_dot_q8k(int type, int bytes, const uint8_t* x, const uint8_t* y, int64_t nb) {
  Levels L;
  double sum = 0.0;
  for (int64_t i = 0; i < nb; ++i) {
    unpack_levels(type, x + i * bytes, &L);
    sum += block_dot_q8k(L, y + i * 292);
  }
  return sum;
}

}  // namespace

extern "C" {

int pm_gguf_block_elems(int type) { const Fmt* f = find_fmt(type); return f ? f->elems : 0; }
int pm_gguf_block_bytes(int type) { const Fmt* f = find_fmt(type); return f ? f->bytes : 0; }
int64_t pm_gguf_row_bytes(int type, int64_t n) {
  const Fmt* f = find_fmt(type);
  return f ? (n + f->elems - 1) / f->elems * f->bytes : -1;
}

int pm_gguf_quantize(int type, const float* src, void* dst, int64_t n, int threads) {
  const Fmt* f = find_fmt(type);
  if (!f) return -1;
  uint8_t* out = static_cast<uint8_t*>(dst);
  if (type == T_F32) { std::memcpy(out, src, static_cast<size_t>(n) * 4); return 0; }
  if (type == T_F16 || type == T_BF16) {
    parallel_blocks(n, threads * 64, [&](int64_t a, int64_t b) {
      for (int64_t i = a; i < b; ++i) put16(out + 2 * i, type == T_F16 ? f32_to_f16(src[i]) : f32_to_bf16(src[i]));
    });
    return 0;
  }
  const EncFn enc = encoder(type);
  if (!enc) return -2;
  const int64_t nb = (n + f->elems - 1) / f->elems;
  const bool k_quant = type >= T_Q2K && type <= T_Q8K;   // only these leave a ragged tail block zeroed; the rest pad
  parallel_blocks(nb, threads, [&](int64_t a, int64_t b) {
    for (int64_t i = a; i < b; ++i) {
      const int64_t left = n - i * f->elems;
      uint8_t* o = out + i * f->bytes;
      if (left >= f->elems) enc(src + i * f->elems, f->elems, o);
      else if (k_quant) std::memset(o, 0, static_cast<size_t>(f->bytes));   // ragged K-quant tail stays zero
      else enc(src + i * f->elems, static_cast<int>(left), o);
    }
  });
  return 0;
}

int pm_gguf_dequantize(int type, const void* src, float* dst, int64_t n, int threads) {
  const Fmt* f = find_fmt(type);
  if (!f) return -1;
  const uint8_t* in = static_cast<const uint8_t*>(src);
  if (type == T_F32) { std::memcpy(dst, in, static_cast<size_t>(n) * 4); return 0; }
  if (type == T_F16 || type == T_BF16) {
    for (int64_t i = 0; i < n; ++i) {
      if (type == T_F16) { dst[i] = f16_to_f32(get16(in + 2 * i)); }
      else { const uint32_t w = static_cast<uint32_t>(get16(in + 2 * i)) << 16; std::memcpy(dst + i, &w, 4); }
    }
    return 0;
  }
  const DecFn dec = decoder(type);
  if (!dec) return -2;
  const int64_t nb = (n + f->elems - 1) / f->elems;
  parallel_blocks(nb, threads, [&](int64_t a, int64_t b) {
    float tmp[256];
    for (int64_t i = a; i < b; ++i) {
      const int64_t left = n - i * f->elems;
      if (left >= f->elems) { dec(in + i * f->bytes, dst + i * f->elems); }
      else { dec(in + i * f->bytes, tmp); std::memcpy(dst + i * f->elems, tmp, static_cast<size_t>(left) * 4); }
    }
  });
  return 0;
}

// x: n elements of a K-quant type (Q2_K..Q6_K, Q8_K); y: the same n elements quantised as Q8_K. n must be a
// multiple of 256. Returns 0 and the dot product in *out; -1 unknown type, -2 type without an integer path, -3 bad n.
int pm_gguf_vec_dot_q8k(int type, const void* x, const void* y_q8k, int64_t n, float* out) {
  const Fmt* f = find_fmt(type);
  if (!f) return -1;
  if (!(type >= T_Q2K && type <= T_Q8K)) return -2;
  if (n <= 0 || n % 256) return -3;
  *out = static_cast<float>(row_dot_q8k(type, f->bytes, static_cast<const uint8_t*>(x),
                                        static_cast<const uint8_t*>(y_q8k), n / 256));
  return 0;
}

// out[r] = dot(W[r, :], y) for a row-major quantised matrix W [rows, n] (rows split over threads).
int pm_gguf_matvec_q8k(int type, const void* w, int64_t rows, int64_t n, const void* y_q8k, float* out, int threads) {
  const Fmt* f = find_fmt(type);
  if (!f) return -1;
  if (!(type >= T_Q2K && type <= T_Q8K)) return -2;
  if (n <= 0 || n % 256 || rows < 0) return -3;
  const int64_t nb = n / 256, row_bytes = nb * f->bytes;
  const uint8_t* W = static_cast<const uint8_t*>(w);
  const uint8_t* y = static_cast<const uint8_t*>(y_q8k);
  parallel_blocks(rows, threads, [&](int64_t a, int64_t b) {
    for (int64_t r = a; r < b; ++r) out[r] = static_cast<float>(row_dot_q8k(type, f->bytes, W + r * row_bytes, y, nb));
  });
  return 0;
}

}  // extern "C"
