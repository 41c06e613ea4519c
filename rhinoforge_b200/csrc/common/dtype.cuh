// 16-bit float helpers shared by the kernels (fp16 and bf16 instantiations).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace rf {

enum DType : int32_t { kF16 = 0, kBF16 = 1, kF32 = 2, kI8 = 3 };

template <typename T> struct Num;
template <> struct Num<__half> {
  static constexpr int kFmt = 0;
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float2 to_f2(__half2 v) { return __half22float2(v); }
  static __device__ __forceinline__ __half2 from_f2(float a, float b) {
    return __floats2half2_rn(a, b);
  }
};
template <> struct Num<__nv_bfloat16> {
  static constexpr int kFmt = 1;
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) {
    return __float2bfloat16_rn(v);
  }
  static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 v) {
    return __bfloat1622float2(v);
  }
  static __device__ __forceinline__ __nv_bfloat162 from_f2(float a, float b) {
    return __floats2bfloat162_rn(a, b);
  }
};

// 8 x 16-bit values in one 16-byte register quad.
template <typename T> struct alignas(16) Vec8 {
  typename Num<T>::T2 v[4];
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  Vec8<T> x = *reinterpret_cast<const Vec8<T>*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = Num<T>::to_f2(x.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  Vec8<T> x;
#pragma unroll
  for (int i = 0; i < 4; ++i) x.v[i] = Num<T>::from_f2(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<Vec8<T>*>(p) = x;
}

// Activations run inside GEMM epilogues whose instruction count is on the critical path (the epilogue warps
// share schedulers with the MMA-issuing lane), so they use the approximate special-function units: results are
// rounded to 16 bits afterwards and the approximation error (2^-11 relative for tanh, 2 ulp for the division)
// is below that rounding.
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float tanh_approx_f(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanh_approx_f(u));
}
__device__ __forceinline__ float gelu_erf_f(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
}

enum Act : int32_t {
  kActNone = 0,
  kActSiluMul = 1,      // dual accumulator: silu(g) * u
  kActGeluTanhMul = 2,  // dual accumulator: gelu_tanh(g) * u
  kActGeluTanh = 3,
  kActGeluErf = 4,
  kActSilu = 5,
};

__device__ __forceinline__ float apply_act(int act, float g, float u) {
  switch (act) {
    case kActSiluMul: return silu_f(g) * u;
    case kActGeluTanhMul: return gelu_tanh_f(g) * u;
    case kActGeluTanh: return gelu_tanh_f(g);
    case kActGeluErf: return gelu_erf_f(g);
    case kActSilu: return silu_f(g);
    default: return g;
  }
}

// Eight int8 values (two 32-bit words) -> eight 16-bit floats, exactly.
// fp16: byte b = x + 128 is dropped into the mantissa of 1024.0 (0x6400 | b = 1024 + b), then 1152 is
// subtracted -- two integer permutes and one half2 subtract per four values, no int->float convert.
template <typename T> __device__ __forceinline__ uint4 widen_i8x8(uint2 q);
template <> __device__ __forceinline__ uint4 widen_i8x8<__half>(uint2 q) {
  const uint32_t bias = 0x64806480u;  // half2(1152, 1152)
  uint4 r;
  uint32_t x = q.x ^ 0x80808080u;
  uint32_t lo = __byte_perm(x, 0x64646464u, 0x5140), hi = __byte_perm(x, 0x64646464u, 0x5342);
  __half2 a = __hsub2(*reinterpret_cast<__half2*>(&lo), *reinterpret_cast<const __half2*>(&bias));
  __half2 b = __hsub2(*reinterpret_cast<__half2*>(&hi), *reinterpret_cast<const __half2*>(&bias));
  r.x = *reinterpret_cast<uint32_t*>(&a);
  r.y = *reinterpret_cast<uint32_t*>(&b);
  x = q.y ^ 0x80808080u;
  lo = __byte_perm(x, 0x64646464u, 0x5140);
  hi = __byte_perm(x, 0x64646464u, 0x5342);
  a = __hsub2(*reinterpret_cast<__half2*>(&lo), *reinterpret_cast<const __half2*>(&bias));
  b = __hsub2(*reinterpret_cast<__half2*>(&hi), *reinterpret_cast<const __half2*>(&bias));
  r.z = *reinterpret_cast<uint32_t*>(&a);
  r.w = *reinterpret_cast<uint32_t*>(&b);
  return r;
}
template <> __device__ __forceinline__ uint4 widen_i8x8<__nv_bfloat16>(uint2 q) {
  const int8_t* b = reinterpret_cast<const int8_t*>(&q);
  uint4 r;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn((float)b[0], (float)b[1]); r.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn((float)b[2], (float)b[3]); r.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn((float)b[4], (float)b[5]); r.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn((float)b[6], (float)b[7]); r.w = *reinterpret_cast<uint32_t*>(&t);
  return r;
}


// Eight int4 values (two's complement nibbles; nibble j of the word holds column {0,2,4,6,1,3,5,7}[j] of the group,
// so that nibbles j and j + 4 are a pair of neighbouring columns) -> eight 16-bit values times `s`, in column order.
// A nibble n becomes the offset code v = n ^ 8 = q + 8 dropped into the mantissa of a power of two (fp16 1024, bf16
// 128: both hold v exactly), from which the offset is subtracted: no integer-to-float conversion.
template <typename T> __device__ __forceinline__ uint4 widen_i4x8(uint32_t x, T s);
template <> __device__ __forceinline__ uint4 widen_i4x8<__half>(uint32_t x, __half s) {
  x ^= 0x88888888u;
  const __half2 off = __half2half2(__float2half_rn(1032.f)), s2 = __half2half2(s);
  uint4 r;
  uint32_t* o = &r.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t t = ((x >> (4 * j)) & 0x000F000Fu) | 0x64006400u;
    __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t), off), s2);
    o[j] = *reinterpret_cast<uint32_t*>(&v);
  }
  return r;
}
template <> __device__ __forceinline__ uint4 widen_i4x8<__nv_bfloat16>(uint32_t x, __nv_bfloat16 s) {
  x ^= 0x88888888u;
  const __nv_bfloat162 off = __bfloat162bfloat162(__float2bfloat16_rn(136.f)), s2 = __bfloat162bfloat162(s);
  uint4 r;
  uint32_t* o = &r.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t t = ((x >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
    __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&t), off), s2);
    o[j] = *reinterpret_cast<uint32_t*>(&v);
  }
  return r;
}

// Eight e2m1 codes (same nibble order as widen_i4x8) -> eight 16-bit values times `s`.  The magnitude index picks a byte
// out of an eight-entry table with one byte permute per four codes (fp16: only the high byte of {0, .5, 1, 1.5, 2, 3, 4,
// 6} is non-zero); the sign bit of the code moves to the sign bit of the value.
template <typename T> __device__ __forceinline__ uint4 widen_e2m1x8(uint32_t x, T s);
template <> __device__ __forceinline__ uint4 widen_e2m1x8<__half>(uint32_t x, __half s) {
  const uint32_t m = x & 0x77777777u;
  const uint32_t a = __byte_perm(0x3E3C3800u, 0x46444240u, m & 0xFFFFu);     // high bytes of codes 0..3
  const uint32_t b = __byte_perm(0x3E3C3800u, 0x46444240u, m >> 16);         // high bytes of codes 4..7
  const __half2 s2 = __half2half2(s);
  uint4 r;
  uint32_t* o = &r.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t t = (((a >> (8 * j)) & 0xFFu) << 8) | (((b >> (8 * j)) & 0xFFu) << 24) | (((x >> (4 * j)) & 0x00080008u) << 12);
    __half2 v = __hmul2(*reinterpret_cast<__half2*>(&t), s2);
    o[j] = *reinterpret_cast<uint32_t*>(&v);
  }
  return r;
}
template <> __device__ __forceinline__ uint4 widen_e2m1x8<__nv_bfloat16>(uint32_t x, __nv_bfloat16 s) {
  const uint32_t m = x & 0x77777777u;
  // bf16 of the eight magnitudes: 0000 3F00 3F80 3FC0 4000 4040 4080 40C0
  const uint32_t ah = __byte_perm(0x3F3F3F00u, 0x40404040u, m & 0xFFFFu), al = __byte_perm(0xC0800000u, 0xC0804000u, m & 0xFFFFu);
  const uint32_t bh = __byte_perm(0x3F3F3F00u, 0x40404040u, m >> 16), bl = __byte_perm(0xC0800000u, 0xC0804000u, m >> 16);
  const __nv_bfloat162 s2 = __bfloat162bfloat162(s);
  uint4 r;
  uint32_t* o = &r.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t t = ((al >> (8 * j)) & 0xFFu) | (((ah >> (8 * j)) & 0xFFu) << 8) | (((bl >> (8 * j)) & 0xFFu) << 16) |
                 (((bh >> (8 * j)) & 0xFFu) << 24) | (((x >> (4 * j)) & 0x00080008u) << 12);
    __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&t), s2);
    o[j] = *reinterpret_cast<uint32_t*>(&v);
  }
  return r;
}

// The same on N values with the activation switch outside the element loop.
template <int N>
__device__ __forceinline__ void apply_act_n(int act, const float (&g)[N], const float (&u)[N], float (&v)[N]) {
  switch (act) {
    case kActSiluMul:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = silu_f(g[j]) * u[j];
      break;
    case kActGeluTanhMul:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = gelu_tanh_f(g[j]) * u[j];
      break;
    case kActGeluTanh:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = gelu_tanh_f(g[j]);
      break;
    case kActGeluErf:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = gelu_erf_f(g[j]);
      break;
    case kActSilu:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = silu_f(g[j]);
      break;
    default:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = g[j];
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace rf
