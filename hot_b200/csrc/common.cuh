// Shared device/host helpers of the HOT B200 kernels: status plumbing, the Philox4x32-10
// counter-based generator, and the per-element quantiser arithmetic.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

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

// Function attributes (the dynamic shared-memory limit) belong to a device, and host threads may
// reach a launcher's first call together: one flag per device ordinal per kernel instantiation.
// Setting an attribute twice is harmless, so the flag only has to be published after the call.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  std::atomic<unsigned char> done[kMaxDevices];
  // Returns the current device ordinal (or -1 on error) and whether it was already marked.
  int current(bool* was_done) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    *was_done = done[dev].load(std::memory_order_acquire) != 0;
    return dev;
  }
  void mark(int dev) { done[dev].store(1, std::memory_order_release); }
};

// ---- quantiser parameters as the kernels see them -------------------------------------
struct QuantDev {
  float qmax;          // 2^(bits-1) - 1
  const float* noise;  // explicit uniforms (ROUND_NOISE)
  uint32_t k0, k1;     // Philox key   = seed
  uint32_t o0, o1;     // Philox c2,c3 = offset
  uint32_t rk0[10], rk1[10];  // the key of each round (the key schedule is the same for every block)
};

inline QuantDev make_quant_dev(const hot_quant_t& q) {
  QuantDev d;
  d.qmax = (float)((1 << (q.bits - 1)) - 1);
  d.noise = q.noise;
  d.k0 = (uint32_t)q.seed;
  d.k1 = (uint32_t)(q.seed >> 32);
  d.o0 = (uint32_t)q.offset;
  d.o1 = (uint32_t)(q.offset >> 32);
  for (int r = 0; r < 10; ++r) {
    d.rk0[r] = d.k0 + (uint32_t)r * 0x9E3779B9u;
    d.rk1[r] = d.k1 + (uint32_t)r * 0xBB67AE85u;
  }
  return d;
}

#ifdef __CUDACC__

constexpr float kEps = 1e-11f;  // the reference's args.eps, added to the scale before dividing

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
// rk0 / rk1: the ten round keys (key + r * Weyl constant), precomputed by the host so that they
// reach the XORs as kernel-parameter operands; each round is two 32 x 32 -> 64 bit products.
__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                               const uint32_t (&rk0)[10], const uint32_t (&rk1)[10]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * (uint64_t)c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * (uint64_t)c2;
    c0 = (uint32_t)(p1 >> 32) ^ c1 ^ rk0[r];
    c1 = (uint32_t)p1;
    c2 = (uint32_t)(p0 >> 32) ^ c3 ^ rk1[r];
    c3 = (uint32_t)p0;
  }
  return make_uint4(c0, c1, c2, c3);
}

// The 16 random bytes of Philox block g: the stochastic-rounding bits of elements 16g .. 16g+15
// (element 16g + j takes byte j, little-endian within the words x, y, z, w).
__device__ __forceinline__ uint4 philox_block16(const QuantDev& q, uint64_t g) {
  return philox4x32_10((uint32_t)g, (uint32_t)(g >> 32), q.o0, q.o1, q.rk0, q.rk1);
}
__device__ __forceinline__ uint32_t philox_byte(const uint4& r, int j) {
  const uint32_t w = j < 4 ? r.x : (j < 8 ? r.y : (j < 12 ? r.z : r.w));
  return (w >> (8 * (j & 3))) & 0xFFu;
}

// ---- packed fp32 (two IEEE round-to-nearest operations per instruction on sm_100) -------
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 sub2(float2 a, float2 b) {
  return __ffma2_rn(b, make_float2(-1.0f, -1.0f), a);  // a - b: the product is exact, one rounding
}

// x / d, correctly rounded, for a divisor shared by many elements: q0 = RN(x * r) with
// r = RN(1 / d), residual e = x - q0 * d (exact in an FMA), q = RN(q0 + e * r).  Equal to IEEE
// division for the ranges a quantiser sees (|x| <= absmax, d = absmax / qmax + eps); the parity
// tests compare against true division bit for bit.
struct Divisor {
  float d;  // the divisor
  float r;  // RN(1 / d)
};

__device__ __forceinline__ Divisor make_divisor(float d) {
  Divisor v;
  v.d = d;
  v.r = __frcp_rn(d);
  return v;
}

__device__ __forceinline__ float div_exact(float x, const Divisor& v) {
  const float q0 = __fmul_rn(x, v.r);
  const float e = __fmaf_rn(-q0, v.d, x);
  return __fmaf_rn(e, v.r, q0);
}

__device__ __forceinline__ float2 div2_exact(float2 x, const Divisor& v) {
  const float2 r2 = make_float2(v.r, v.r), nd2 = make_float2(-v.d, -v.d);
  const float2 q0 = __fmul2_rn(x, r2);
  const float2 e = __ffma2_rn(q0, nd2, x);
  return __ffma2_rn(e, r2, q0);
}

// Everything a quantiser derives from an abs-max: the scale s = mx / qmax the caller gets back,
// the divisor s + eps (fp32, round-to-nearest: the reference divides, it does not multiply by
// a reciprocal), and the constant of the Philox rounding path.
struct ScalePair {
  float s;
  Divisor dv;  // divide by s + eps
  float c0;    // (qmax + 1) - 128 + 1/512, see philox_offset_code
};

__device__ __forceinline__ ScalePair scale_from_absmax(float mx, float qmax) {
  ScalePair p;
  p.s = __fdiv_rn(mx, qmax);
  p.dv = make_divisor(__fadd_rn(p.s, kEps));
  p.c0 = (qmax + 1.0f) - 128.0f + 0.001953125f;  // exact in fp32
  return p;
}

// Philox-path stochastic rounding.  With y = x / d, B = qmax + 1 and R the element's random byte,
//     offset code = floor( y + B + (R + 0.5) / 256 )        (code = offset code - B)
// evaluated as  t1 = RN(y + c0),  t2 = t1 + u  (exact),  floor(t2),  where u = 128 + R / 256 is built
// by dropping R into the mantissa of 128.0f and c0 = B - 128 + 1/512.  The value is shifted to be
// positive so that floor is the rounding for both signs; adding a uniform in (0, 1) and flooring
// rounds up with probability frac(y) to within 1/256, and the +0.5 centres it (no bias).  Since
// |y| <= qmax * (1 + 2^-22), the offset code stays in [1, 2 * qmax + 1]: no clamp needed.
__device__ __forceinline__ float philox_u128(uint32_t word, int byte) {
  return __uint_as_float(__byte_perm(word, 0x43000000u, 0x7404u | ((uint32_t)byte << 4)));
}
constexpr float kFloorMagic = 8388608.0f;  // 2^23: RD(t + 2^23) keeps floor(t) in the low mantissa bits

__device__ __forceinline__ uint32_t philox_offset_code(float x, const ScalePair& sp, float u128) {
  const float t2 = __fadd_rn(__fadd_rn(div_exact(x, sp.dv), sp.c0), u128);
  return __float_as_uint(__fadd_rd(t2, kFloorMagic)) & 0xFFu;
}
// two values at once; returns the raw bits whose low bytes are the offset codes
__device__ __forceinline__ float2 philox_offset_bits2(float2 x, const ScalePair& sp, float2 u128) {
  const float2 t2 = add2(add2(div2_exact(x, sp.dv), make_float2(sp.c0, sp.c0)), u128);
  return __fadd2_rd(t2, make_float2(kFloorMagic, kFloorMagic));
}
// low bytes of four words -> one word
__device__ __forceinline__ uint32_t gather_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040u), __byte_perm(c, d, 0x0040u), 0x5410u);
}
// Packed INT4 layout: a run of 16 codes takes 8 bytes; byte j holds code j in its low nibble and code
// j + 8 in its high nibble.  lo / hi: four byte-wide codes (each < 16) of the first / second half.
__device__ __forceinline__ uint32_t pack_nibbles(uint32_t lo, uint32_t hi) { return lo | (hi << 4); }
// Remove the offset 2^(bits-1) from packed offset codes (a flip of that bit per lane) and
// sign-extend codes narrower than their lane.  lanes: 0x11111111 (nibbles) or 0x01010101 (bytes).
__device__ __forceinline__ uint32_t remove_offset(uint32_t w, uint32_t off, uint32_t lanes, uint32_t lane_span) {
  w ^= off * lanes;
  const uint32_t ext = lane_span - 2u * off;  // the bits above the sign bit (0 if the code fills its lane)
  if (ext) w |= ((w & (off * lanes)) / off) * ext;
  return w;
}

// One code for the deterministic and the explicit-noise modes, |code| <= qmax.
//   nearest : round-half-even of y = x / d (torch.round)
//   noise   : sign(y) * (floor|y| + [u < frac|y|]) with the caller's uniform u
template <int ROUND>
__device__ __forceinline__ int quantise_one(float x, const ScalePair& sp, float u, int qmax) {
  if (ROUND == HOT_ROUND_NEAREST) {
    const int c = __float2int_rn(div_exact(x, sp.dv));
    return max(-qmax, min(qmax, c));
  }
  const float a = fabsf(div_exact(x, sp.dv));
  const float f = floorf(a);
  int mag = (int)f + ((u < __fsub_rn(a, f)) ? 1 : 0);
  mag = min(mag, qmax);  // the abs-max element can land an ulp above qmax and round up
  return (x < 0.0f) ? -mag : mag;
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
