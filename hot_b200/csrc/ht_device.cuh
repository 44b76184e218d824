// Device helpers shared by the transform + quantise kernels: 16-element runs held as eight
// packed fp32 pairs (A_i, B_i), the order-n butterfly on them, and their quantisation.
#pragma once

#include "common.cuh"

namespace hot {

// ---- loads: 16 consecutive elements -> eight (A_i, B_i) pairs ----------------------------
template <typename T>
struct Load16;
template <>
struct Load16<float> {
  static __device__ __forceinline__ void run(const float* p, float2 (&v)[8]) {
    const float4* q = reinterpret_cast<const float4*>(p);
    const float4 a0 = __ldg(q), a1 = __ldg(q + 1), b0 = __ldg(q + 2), b1 = __ldg(q + 3);
    v[0] = make_float2(a0.x, b0.x); v[1] = make_float2(a0.y, b0.y);
    v[2] = make_float2(a0.z, b0.z); v[3] = make_float2(a0.w, b0.w);
    v[4] = make_float2(a1.x, b1.x); v[5] = make_float2(a1.y, b1.y);
    v[6] = make_float2(a1.z, b1.z); v[7] = make_float2(a1.w, b1.w);
  }
};
template <>
struct Load16<__nv_bfloat16> {
  static __device__ __forceinline__ void run(const __nv_bfloat16* p, float2 (&v)[8]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
    const uint4 a = __ldg(q), b = __ldg(q + 1);
    const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[2 * k] = make_float2(__uint_as_float(wa[k] << 16), __uint_as_float(wb[k] << 16));
      v[2 * k + 1] = make_float2(__uint_as_float(wa[k] & 0xFFFF0000u), __uint_as_float(wb[k] & 0xFFFF0000u));
    }
  }
};

__device__ __forceinline__ void zero16(float2 (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = make_float2(0.0f, 0.0f);
}

// Order-n transform of the 16-element run (n <= 16 entirely in registers, 32 and 64 with the
// neighbouring lanes).  Must be executed by all 32 lanes when n > 16.
__device__ __forceinline__ void butterfly16(float2 (&v)[8], int n, int lane) {
  if (n >= 2) {
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const float2 a = v[i], b = v[i + 1];
      v[i] = add2(a, b);
      v[i + 1] = sub2(a, b);
    }
  }
  if (n >= 4) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & 2) == 0) {
        const float2 a = v[i], b = v[i + 2];
        v[i] = add2(a, b);
        v[i + 2] = sub2(a, b);
      }
    }
  }
  if (n >= 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = v[i], b = v[i + 4];
      v[i] = add2(a, b);
      v[i + 4] = sub2(a, b);
    }
  }
  if (n >= 16) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = make_float2(__fadd_rn(v[i].x, v[i].y), __fsub_rn(v[i].x, v[i].y));
  }
  for (int h = 16; h < n; h <<= 1) {
    const int m = h >> 4;
    const float sg = (lane & m) ? -1.0f : 1.0f;  // upper half: partner - mine; lower: mine + partner
    const float2 sg2 = make_float2(sg, sg);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float2 o;
      o.x = __shfl_xor_sync(0xFFFFFFFFu, v[i].x, m);
      o.y = __shfl_xor_sync(0xFFFFFFFFu, v[i].y, m);
      v[i] = __ffma2_rn(v[i], sg2, o);  // exact product, one rounding: o +- mine
    }
  }
}

// Even rows of the order-16 butterfly over tokens for a channel pair: u[t] = (x[t][c], x[t][c+1]).
// Stage h = 1 leaves the sums x[2i] + x[2i+1] at the even positions, and the later stages only
// ever combine positions of equal parity, so the even outputs need the sums alone: e[i] is
// natural row 2i.  Same operations, in the same order, as the full butterfly computes for them.
__device__ __forceinline__ void butterfly_tokens16_even(const float2 (&u)[16], float2 (&e)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = add2(u[2 * i], u[2 * i + 1]);
#pragma unroll
  for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & h) == 0) {
        const float2 a = e[i], b = e[i + h];
        e[i] = add2(a, b);
        e[i + h] = sub2(a, b);
      }
    }
  }
}

__device__ __forceinline__ float absmax16(const float2 (&v)[8]) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fmaxf(fabsf(v[i].x), fabsf(v[i].y)));
  return m;
}

// Quantise the 16 transformed values whose first logical element index is `e0` (a multiple of
// 16) and store them at `dst` (8 bytes for INT4, 16 for INT8).
template <int ROUND, int STORE4>
__device__ __forceinline__ void quantise_store16(const float2 (&v)[8], const ScalePair& sp, const QuantDev& q, uint64_t e0,
                                                 uint8_t* dst) {
  uint32_t wa0 = 0, wa1 = 0, wb0 = 0, wb1 = 0;  // INT4: wa0 = A, wb0 = B; INT8: (wa0, wa1) = A, (wb0, wb1) = B
  if (ROUND == HOT_ROUND_STOCH_PHILOX) {
    const bool rb4 = rand_bits(q.qmax) == 4;
    const float2 mk2 = make_float2(sp.mk, sp.mk), ck2 = make_float2(sp.ck, sp.ck);
    uint32_t ka[8], kb[8];  // raw bits of RN(x * mk + ck); the low mantissa bits are K
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 t = __ffma2_rn(v[i], mk2, ck2);
      ka[i] = __float_as_uint(t.x);
      kb[i] = __float_as_uint(t.y);
    }
    philox_run16(ka, kb, q, e0, rb4, wa0, wa1, wb0, wb1);
    const uint32_t off = (uint32_t)(q.qmax + 1.0f);
    if (STORE4) {  // (always 4 random bits) element i is code i, element i + 8 code i + 8: byte i = code i | code (i + 8) << 4
      const uint32_t p0 = remove_offset(((wa0 >> 4) & 0x0F0F0F0Fu) | (wb0 & 0xF0F0F0F0u), off, 0x11111111u, 0x10u);
      const uint32_t p1 = remove_offset(((wa1 >> 4) & 0x0F0F0F0Fu) | (wb1 & 0xF0F0F0F0u), off, 0x11111111u, 0x10u);
      wa0 = p0;
      wb0 = p1;
    } else {
      if (rb4) {
        wa0 = (wa0 >> 4) & 0x0F0F0F0Fu; wa1 = (wa1 >> 4) & 0x0F0F0F0Fu;
        wb0 = (wb0 >> 4) & 0x0F0F0F0Fu; wb1 = (wb1 >> 4) & 0x0F0F0F0Fu;
      }
      wa0 = remove_offset(wa0, off, 0x01010101u, 0x100u);
      wa1 = remove_offset(wa1, off, 0x01010101u, 0x100u);
      wb0 = remove_offset(wb0, off, 0x01010101u, 0x100u);
      wb1 = remove_offset(wb1, off, 0x01010101u, 0x100u);
    }
  } else {
    float ua[8], ub[8];
    if (ROUND == HOT_ROUND_STOCH_NOISE) {
      Load8<float>::run(q.noise + e0, ua);
      Load8<float>::run(q.noise + e0 + 8, ub);
    }
    const int qmax = (int)q.qmax;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int ca = quantise_one<ROUND>(v[i].x, sp, ROUND == HOT_ROUND_STOCH_NOISE ? ua[i] : 0.0f, qmax);
      const int cb = quantise_one<ROUND>(v[i].y, sp, ROUND == HOT_ROUND_STOCH_NOISE ? ub[i] : 0.0f, qmax);
      if (STORE4) {  // byte i = code i | code (i + 8) << 4; bytes 0..3 in wa0, 4..7 in wb0
        const uint32_t byte = (uint32_t)(ca & 0xF) | ((uint32_t)(cb & 0xF) << 4);
        if (i < 4) wa0 |= byte << (8 * i);
        else wb0 |= byte << (8 * (i - 4));
      } else {
        if (i < 4) { wa0 |= (uint32_t)(ca & 0xFF) << (8 * i); wb0 |= (uint32_t)(cb & 0xFF) << (8 * i); }
        else { wa1 |= (uint32_t)(ca & 0xFF) << (8 * (i - 4)); wb1 |= (uint32_t)(cb & 0xFF) << (8 * (i - 4)); }
      }
    }
  }
  if (STORE4) *reinterpret_cast<uint2*>(dst) = make_uint2(wa0, wb0);
  else *reinterpret_cast<uint4*>(dst) = make_uint4(wa0, wa1, wb0, wb1);
}

}  // namespace hot
