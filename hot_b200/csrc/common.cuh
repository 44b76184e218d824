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

// Philox4x32 rounds.  Salmon et al. ("Parallel random numbers: as easy as 1, 2, 3") give 10 as the
// default and 7 as the fewest rounds that pass BigCrush; the rounding bits of a quantiser need no
// more than that, and three rounds fewer are a third of the generator's integer work.
constexpr int kPhiloxRounds = 7;

// The layer's weight [O, I] (dtype, O and transform order of the grad_out it goes with), transformed along O and
// quantised with one scale by the tensor-core grad_out kernels on the side: codes [I, O] one per byte at pitch
// ld_qw, scale to s_w[0]; max_w is one scratch word (cleared by the call).
struct TcWeightJob {
  const void* w;
  int64_t ldw, I;
  hot_quant_t q;
  void* q_w;
  int64_t ld_qw;
  float* s_w;
  uint32_t* max_w;
};

// ---- quantiser parameters as the kernels see them -------------------------------------
struct QuantDev {
  float qmax;          // 2^(bits-1) - 1
  const float* noise;  // explicit uniforms (ROUND_NOISE)
  uint32_t k0, k1;     // Philox key   = seed
  uint32_t o0, o1;     // Philox c2,c3 = offset
  uint32_t rk0[kPhiloxRounds], rk1[kPhiloxRounds];  // the key of each round (the key schedule is the same for every block)
};

inline QuantDev make_quant_dev(const hot_quant_t& q) {
  QuantDev d;
  d.qmax = (float)((1 << (q.bits - 1)) - 1);
  d.noise = q.noise;
  d.k0 = (uint32_t)q.seed;
  d.k1 = (uint32_t)(q.seed >> 32);
  d.o0 = (uint32_t)q.offset;
  d.o1 = (uint32_t)(q.offset >> 32);
  for (int r = 0; r < kPhiloxRounds; ++r) {
    d.rk0[r] = d.k0 + (uint32_t)r * 0x9E3779B9u;
    d.rk1[r] = d.k1 + (uint32_t)r * 0xBB67AE85u;
  }
  return d;
}

#ifdef __CUDACC__

constexpr float kEps = 1e-11f;  // the reference's args.eps, added to the scale before dividing

// Philox4x32 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"), kPhiloxRounds rounds.
// rk0 / rk1: the round keys (key + r * Weyl constant), precomputed by the host so that they
// reach the XORs as kernel-parameter operands; each round is two 32 x 32 -> 64 bit products.
__device__ __forceinline__ uint4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                            const uint32_t (&rk0)[kPhiloxRounds], const uint32_t (&rk1)[kPhiloxRounds]) {
#pragma unroll
  for (int r = 0; r < kPhiloxRounds; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * (uint64_t)c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * (uint64_t)c2;
    c0 = (uint32_t)(p1 >> 32) ^ c1 ^ rk0[r];
    c1 = (uint32_t)p1;
    c2 = (uint32_t)(p0 >> 32) ^ c3 ^ rk1[r];
    c3 = (uint32_t)p0;
  }
  return make_uint4(c0, c1, c2, c3);
}

// Philox block g: counter (g_lo, g_hi, offset_lo, offset_hi), key = seed.  Which elements a block
// serves depends on the random bits a code takes (rand_bits below):
//   8 bits: elements 16g .. 16g+15; element 16g + j takes byte j % 4 (little-endian) of word j / 4
//   4 bits: elements 32g .. 32g+31; with j = e % 32, run h = j / 16, i = j % 16, element e takes
//           nibble i / 8 of byte i % 4 of word 2h + (i % 8) / 4, so that one word serves elements
//           i..i+3 of a run with its low nibbles and i+8..i+11 with its high ones
__device__ __forceinline__ uint4 philox_block(const QuantDev& q, uint64_t g) {
  return philox4x32((uint32_t)g, (uint32_t)(g >> 32), q.o0, q.o1, q.rk0, q.rk1);
}
__device__ __forceinline__ uint32_t philox_word(const uint4& r, int w) {
  return w == 0 ? r.x : (w == 1 ? r.y : (w == 2 ? r.z : r.w));
}
// the 8-bit / 4-bit random number of stored-layout element e, from the block that serves it
__device__ __forceinline__ uint32_t philox_r8(const uint4& blk, uint64_t e) {
  const int j = (int)(e & 15u);
  return (philox_word(blk, j >> 2) >> (8 * (j & 3))) & 0xFFu;
}
__device__ __forceinline__ uint32_t philox_r4(const uint4& blk, uint64_t e) {
  const int i = (int)(e & 15u), h = (int)((e >> 4) & 1u);
  return (philox_word(blk, 2 * h + ((i & 7) >> 2)) >> (8 * (i & 3) + 4 * (i >> 3))) & 0xFu;
}
// the two words of the 16-element run that starts at element e0 (a multiple of 16), 4-bit numbers
__device__ __forceinline__ void philox_run_words4(const QuantDev& q, uint64_t e0, uint32_t& r0, uint32_t& r1) {
  const uint4 b = philox_block(q, e0 >> 5);
  const bool hi = (e0 & 16u) != 0;
  r0 = hi ? b.z : b.x;
  r1 = hi ? b.w : b.y;
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
// a reciprocal), and the constants of the Philox rounding path.
struct ScalePair {
  float s;
  Divisor dv;  // divide by s + eps
  float mk;    // RN(2^RB / (s + eps)), RB = rand_bits(qmax)
  float ck;    // 1.5 * 2^23 + 2^RB * (qmax + 1)
};

// Random bits per code on the Philox path: 4 for codes of up to 4 bits, else 8.
__host__ __device__ __forceinline__ int rand_bits(float qmax) { return qmax <= 7.0f ? 4 : 8; }
constexpr float kKMagic = 12582912.0f;  // 1.5 * 2^23 = 0x4B400000: the low mantissa bits of RN(t + this) are RN(t) as an integer

__device__ __forceinline__ ScalePair scale_from_absmax(float mx, float qmax) {
  ScalePair p;
  p.s = __fdiv_rn(mx, qmax);
  p.dv = make_divisor(__fadd_rn(p.s, kEps));
  const float two_rb = qmax <= 7.0f ? 16.0f : 256.0f;
  p.mk = __fdiv_rn(two_rb, p.dv.d);
  p.ck = kKMagic + two_rb * (qmax + 1.0f);  // exact in fp32
  return p;
}

// Philox-path stochastic rounding.  With RB random bits per code, R the element's RB-bit random
// number, B = qmax + 1 and m = RN(2^RB / d):
//     K = round_half_even(x * m) + 2^RB * B,      offset code = (K + R) >> RB      (code = offset code - B)
// K comes out of ONE fused multiply-add: RN(x * m + (1.5 * 2^23 + 2^RB * B)) lies in [2^23, 2^24), where
// fp32 has unit spacing, so its low mantissa bits are K (x * m enters the rounding exactly).  The
// quotient is thereby rounded to RB fractional bits; adding a uniform RB-bit integer and dropping
// RB bits rounds up with probability round(2^RB * frac) / 2^RB: unbiased.  Since |x * m| <=
// 2^RB * qmax * (1 + 2^-22), K + R stays within [2^RB, 2^RB * (2 * qmax + 2)): no clamp, and for
// RB = 4 / 8 the sum fits an 8- / 16-bit lane, so the random numbers are added to packed lanes.
__device__ __forceinline__ uint32_t philox_kbits(float x, const ScalePair& sp) {
  return __float_as_uint(__fmaf_rn(x, sp.mk, sp.ck));
}
__device__ __forceinline__ uint32_t philox_offset_code(float x, const ScalePair& sp, uint32_t r, int rb) {
  return ((philox_kbits(x, sp) & 0xFFFFu) + r) >> rb;
}
// low bytes of four words -> one word
__device__ __forceinline__ uint32_t gather_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040u), __byte_perm(c, d, 0x0040u), 0x5410u);
}
// Four offset codes (one per byte) of the K words k0..k3 of elements j..j+3 with 8 random bits each:
// rw = the word whose bytes are their random numbers.  Two K values share a 32-bit word in 16-bit lanes.
__device__ __forceinline__ uint32_t offset_codes4_rb8(uint32_t k0, uint32_t k1, uint32_t k2, uint32_t k3, uint32_t rw) {
  const uint32_t s02 = __byte_perm(k0, k2, 0x5410u) + (rw & 0x00FF00FFu);
  const uint32_t s13 = __byte_perm(k1, k3, 0x5410u) + __byte_perm(rw, 0u, 0x4341u);
  return __byte_perm(s02, s13, 0x7351u);
}
// Four sums K + R (one per byte; the offset code is the high nibble) with 4 random bits each:
// rn = the four random nibbles, one per byte, already masked
__device__ __forceinline__ uint32_t offset_sums4_rb4(uint32_t k0, uint32_t k1, uint32_t k2, uint32_t k3, uint32_t rn) {
  return gather_low_bytes(k0, k1, k2, k3) + rn;
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

// The 16 offset codes of a run whose K words are ka[0..7] (elements 0..7) and kb[0..7] (elements
// 8..15), Philox rounding; e0 = stored-layout index of element 0 (a multiple of 16).
//   RB = 4: wa0 / wb0 / wa1 / wb1 hold the sums of elements 0-3 / 8-11 / 4-7 / 12-15 (code = high nibble)
//   RB = 8: they hold the offset codes of those elements, one per byte
__device__ __forceinline__ void philox_run16_words(const uint32_t* ka, const uint32_t* kb, bool rb4, uint32_t r0, uint32_t r1,
                                                   uint32_t r2, uint32_t r3, uint32_t& wa0, uint32_t& wa1, uint32_t& wb0,
                                                   uint32_t& wb1) {
  // rb4: (r0, r1) are the run's two words; else (r0, r1, r2, r3) are the four words of its block
  if (rb4) {
    wa0 = offset_sums4_rb4(ka[0], ka[1], ka[2], ka[3], r0 & 0x0F0F0F0Fu);
    wb0 = offset_sums4_rb4(kb[0], kb[1], kb[2], kb[3], (r0 >> 4) & 0x0F0F0F0Fu);
    wa1 = offset_sums4_rb4(ka[4], ka[5], ka[6], ka[7], r1 & 0x0F0F0F0Fu);
    wb1 = offset_sums4_rb4(kb[4], kb[5], kb[6], kb[7], (r1 >> 4) & 0x0F0F0F0Fu);
  } else {
    wa0 = offset_codes4_rb8(ka[0], ka[1], ka[2], ka[3], r0);
    wa1 = offset_codes4_rb8(ka[4], ka[5], ka[6], ka[7], r1);
    wb0 = offset_codes4_rb8(kb[0], kb[1], kb[2], kb[3], r2);
    wb1 = offset_codes4_rb8(kb[4], kb[5], kb[6], kb[7], r3);
  }
}
__device__ __forceinline__ void philox_run16(const uint32_t* ka, const uint32_t* kb, const QuantDev& q, uint64_t e0,
                                             bool rb4, uint32_t& wa0, uint32_t& wa1, uint32_t& wb0, uint32_t& wb1) {
  if (rb4) {
    uint32_t r0, r1;
    philox_run_words4(q, e0, r0, r1);
    philox_run16_words(ka, kb, true, r0, r1, 0u, 0u, wa0, wa1, wb0, wb1);
  } else {
    const uint4 r = philox_block(q, e0 >> 4);
    philox_run16_words(ka, kb, false, r.x, r.y, r.z, r.w, wa0, wa1, wb0, wb1);
  }
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
