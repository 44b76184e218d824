// Shared device/host helpers of the HOT B200 kernels: status plumbing, the Philox4x32-10
// counter-based generator, and the per-element quantiser arithmetic.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "hot_b200.h"

namespace hot {

// ---- host-side error plumbing ---------------------------------------------------------
void set_error(const char* fmt, ...);
#define HOT_FAIL(code, ...)     \
  do {                          \
    ::hot::set_error(__VA_ARGS__); \
    return (code);              \
  } while (0)
#define HOT_CUDA(expr)                                                              \
  do {                                                                              \
    cudaError_t e_ = (expr);                                                        \
    if (e_ != cudaSuccess) HOT_FAIL(HOT_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

int validate_quant(const hot_quant_t* q, const char* who);

// ---- quantiser parameters as the kernels see them -------------------------------------
struct QuantDev {
  float qmax;          // 2^(bits-1) - 1
  const float* noise;  // explicit uniforms (ROUND_NOISE)
  uint32_t k0, k1;     // Philox key   = seed
  uint32_t o0, o1;     // Philox c2,c3 = offset
};

inline QuantDev make_quant_dev(const hot_quant_t& q) {
  QuantDev d;
  d.qmax = (float)((1 << (q.bits - 1)) - 1);
  d.noise = q.noise;
  d.k0 = (uint32_t)q.seed;
  d.k1 = (uint32_t)(q.seed >> 32);
  d.o0 = (uint32_t)q.offset;
  d.o1 = (uint32_t)(q.offset >> 32);
  return d;
}

#ifdef __CUDACC__

constexpr float kEps = 1e-11f;  // the reference's args.eps, added to the scale before dividing

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                               uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// The eight 16-bit uniforms of Philox block g (elements 8g .. 8g+7), as floats k/65536.
__device__ __forceinline__ void philox_uniform8(const QuantDev& q, uint64_t g, float (&u)[8]) {
  const uint4 w = philox4x32_10((uint32_t)g, (uint32_t)(g >> 32), q.o0, q.o1, q.k0, q.k1);
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    u[2 * i] = (float)(ws[i] & 0xFFFFu) * (1.0f / 65536.0f);
    u[2 * i + 1] = (float)(ws[i] >> 16) * (1.0f / 65536.0f);
  }
}

// scale and divisor of a quantiser from an abs-max: s = mx / qmax, d = s + eps (both fp32,
// IEEE round-to-nearest: the reference divides, it does not multiply by a reciprocal).
__device__ __forceinline__ void scale_from_absmax(float mx, float qmax, float& s, float& d) {
  s = __fdiv_rn(mx, qmax);
  d = __fadd_rn(s, kEps);
}

// One code.  ROUND: hot_rounding.  u is the uniform for stochastic modes.
template <int ROUND>
__device__ __forceinline__ int quantise_one(float x, float d, float u) {
  const float y = __fdiv_rn(x, d);
  if (ROUND == HOT_ROUND_NEAREST) return __float2int_rn(y);  // half to even, as torch.round
  const float a = fabsf(y);
  const float f = floorf(a);
  const float frac = __fsub_rn(a, f);
  int i = (int)f + ((u < frac) ? 1 : 0);
  return (y < 0.0f) ? -i : i;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// Non-negative floats order like their bit patterns, so an unsigned atomicMax works.
__device__ __forceinline__ void atomic_absmax(uint32_t* p, float v) { atomicMax(p, __float_as_uint(v)); }

template <typename T>
struct Load8;
template <>
struct Load8<float> {
  static __device__ __forceinline__ void run(const float* p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <>
struct Load8<__nv_bfloat16> {
  static __device__ __forceinline__ void run(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
};

#endif  // __CUDACC__

}  // namespace hot
