// Fused block Walsh-Hadamard transform along the FIRST dim (with row selection: the Hadamard
// low-rank projection) + INT4/INT8 quantisation, written transposed.
//
// A CTA owns a tile of NB token blocks (NB * n rows) by CC columns.  Phase 1: each warp takes
// whole token blocks; a thread loads its columns of the n rows of a block with warp-coalesced
// 4-byte loads, runs the order-n butterfly in registers (stages h = 1, 2, 4, ... on pairs
// (t, t + h) -> (x + y, x - y), the order the CPU oracle fixes) and drops the kept rows into a
// float tile in shared memory, transposed: tile[column][block * r + j].  Phase 2: threads walk
// the tile rows, 8 consecutive codes each, quantise (one Philox block per 8 codes) and store
// 4 or 8 contiguous bytes, so that rows of the transposed output are written in full sectors.
//
// Per-tensor and per-output-row scales need the abs-max of the transformed tensor first: a
// first launch runs phase 1 only and reduces into the scratch words.
#include "common.cuh"

namespace hot {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

struct ColParams {
  int64_t rows, ldx, ld_codes;
  int cols, r, nb;            // nb: token blocks per tile
  int pitch;                  // floats per tile row
  int64_t out_len;            // rows * r / n
  int scale_row, store4, noise_transposed;
  int sawb;                   // clip from the second moment and the mean magnitude instead of the abs-max
  signed char pos[64];        // pos[k] = output slot of natural row k, or -1
  // batched call (blockIdx.z = sample; rows / out_len are per sample, one scale per sample):
  int batch;                  // 1 in a plain call
  int64_t sample_pitch;       // bytes from one sample's codes to the next within an output row; 0 in a plain call
};

template <typename T>
struct ColTraits;
template <>
struct ColTraits<float> {
  static constexpr int kCpl = 1;  // columns per 4-byte load
  static __device__ __forceinline__ void load(const float* p, bool ok, float (&o)[1]) { o[0] = ok ? __ldg(p) : 0.0f; }
};
template <>
struct ColTraits<__nv_bfloat16> {
  static constexpr int kCpl = 2;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, bool ok, float (&o)[2]) {
    const uint32_t w = ok ? __ldg(reinterpret_cast<const uint32_t*>(p)) : 0u;
    o[0] = __uint_as_float(w << 16);
    o[1] = __uint_as_float(w & 0xFFFF0000u);
  }
};

// A warp handles G consecutive token blocks at a time, G * N = 16 rows for the small orders, so that
// it always has at least 16 independent rows of loads in flight.
template <int N>
__host__ __device__ constexpr int group_for() {
  return N >= 16 ? 1 : 16 / N;
}
// column groups per thread, bounding the register tile at 64 floats (128 for bf16 at n = 64)
template <typename T, int N>
__host__ __device__ constexpr int vec_for() {
  constexpr int rows = N * group_for<N>();
  return (64 / (rows * ColTraits<T>::kCpl)) >= 4 ? 4 : ((64 / (rows * ColTraits<T>::kCpl)) >= 2 ? 2 : 1);
}

// order-N butterfly on v[OFF .. OFF + N)
template <int N, int OFF, int LEN>
__device__ __forceinline__ void butterfly_regs(float (&v)[LEN]) {
#pragma unroll
  for (int h = 1; h < N; h <<= 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if ((i & h) == 0) {
        const float a = v[OFF + i], b = v[OFF + i + h];
        v[OFF + i] = a + b;
        v[OFF + i + h] = a - b;
      }
    }
  }
}
template <int N, int G, int LEN>
__device__ __forceinline__ void butterfly_groups(float (&v)[LEN]) {
  if constexpr (G >= 1) {
    butterfly_regs<N, (G - 1) * N, LEN>(v);
    butterfly_groups<N, G - 1, LEN>(v);
  }
}

// Loads the G blocks starting at `blk` (global block index; blocks at or past nblk read as zeros) for
// this thread's columns and transforms each: v[column][g * N + k] = row k of block blk + g.
template <typename T, int N, int VEC>
__device__ __forceinline__ void load_transform(const T* __restrict__ x, const ColParams& p, int64_t blk, int64_t nblk, int c0,
                                               int lane, float (&v)[VEC * ColTraits<T>::kCpl][N * group_for<N>()]) {
  constexpr int CPL = ColTraits<T>::kCpl;
  constexpr int G = group_for<N>();
  const T* base = x + blk * N * p.ldx;
#pragma unroll
  for (int t = 0; t < N * G; ++t) {
    const bool row_ok = blk + t / N < nblk;
#pragma unroll
    for (int vv = 0; vv < VEC; ++vv) {
      const int c = c0 + (lane + 32 * vv) * CPL;
      float o[CPL];
      ColTraits<T>::load(base + (int64_t)t * p.ldx + c, row_ok && c < p.cols, o);
#pragma unroll
      for (int q = 0; q < CPL; ++q) v[vv * CPL + q][t] = o[q];
    }
  }
#pragma unroll
  for (int i = 0; i < VEC * CPL; ++i) butterfly_groups<N, G, N * G>(v[i]);
}

// ---- pass 1: abs-max of the kept, transformed rows --------------------------------------
template <typename T, int N>
__global__ void __launch_bounds__(kThreads) col_ht_absmax_kernel(const T* __restrict__ x, ColParams p,
                                                                 uint32_t* __restrict__ absmax) {
  constexpr int VEC = vec_for<T, N>();
  constexpr int CPL = ColTraits<T>::kCpl;
  constexpr int CC = 32 * VEC * CPL;
  __shared__ uint32_t s_max[CC];
  x += (int64_t)blockIdx.z * p.rows * p.ldx;
  // SAWB: two doubles per CTA, the CTAs of sample z at (z * gridDim.y + y) * gridDim.x + x
  double* sawb_part = reinterpret_cast<double*>(absmax) + 2 * (((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x);
  absmax += (size_t)blockIdx.z * (p.scale_row ? (size_t)p.cols : 1);  // batched: one abs-max word (or one row of them) per sample
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * CC;
  const int64_t nblk = p.rows / N;
  const int64_t blk0 = (int64_t)blockIdx.y * p.nb;
  for (int i = threadIdx.x; i < CC; i += kThreads) s_max[i] = 0u;
  __syncthreads();
  float cm[VEC * CPL];
#pragma unroll
  for (int i = 0; i < VEC * CPL; ++i) cm[i] = 0.0f;
  double sum_sq = 0.0, sum_abs = 0.0;  // SAWB statistics of this thread
  constexpr int G = group_for<N>();
  for (int b = warp * G; b < p.nb; b += kWarps * G) {
    if (blk0 + b >= nblk) break;
    float v[VEC * CPL][N * G];
    load_transform<T, N, VEC>(x, p, blk0 + b, nblk, c0, lane, v);
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int k = 0; k < N; ++k) {
        if (p.pos[k] >= 0) {
#pragma unroll
          for (int i = 0; i < VEC * CPL; ++i) cm[i] = fmaxf(cm[i], fabsf(v[i][g * N + k]));
          if (p.sawb) {
            // in double throughout (the squares are exact there), so that the two means round to
            // float once, as a float64 mean does; columns and blocks beyond the matrix were loaded as zeros
#pragma unroll
            for (int i = 0; i < VEC * CPL; ++i) {
              const double d = (double)v[i][g * N + k];
              sum_sq = fma(d, d, sum_sq);
              sum_abs += fabs(d);
            }
          }
        }
      }
    }
  }
  if (p.sawb) {
    // one (sum of squares, sum of magnitudes) pair per CTA, reduced in a fixed order; the second
    // pass adds the pairs up in a fixed order too, so the clip value is reproducible
    __shared__ double s_sum[2][kWarps];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sum_sq += __shfl_xor_sync(0xFFFFFFFFu, sum_sq, o);
      sum_abs += __shfl_xor_sync(0xFFFFFFFFu, sum_abs, o);
    }
    if (lane == 0) {
      s_sum[0][warp] = sum_sq;
      s_sum[1][warp] = sum_abs;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      double a = 0.0, b = 0.0;
      for (int w = 0; w < kWarps; ++w) {
        a += s_sum[0][w];
        b += s_sum[1][w];
      }
      sawb_part[0] = a;
      sawb_part[1] = b;
    }
    return;
  }
  if (p.scale_row) {
#pragma unroll
    for (int vv = 0; vv < VEC; ++vv)
#pragma unroll
      for (int q = 0; q < CPL; ++q) atomicMax(&s_max[(lane + 32 * vv) * CPL + q], __float_as_uint(cm[vv * CPL + q]));
    __syncthreads();
    for (int i = threadIdx.x; i < CC; i += kThreads)
      if (c0 + i < p.cols) atomicMax(absmax + c0 + i, s_max[i]);
  } else {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC * CPL; ++i) m = fmaxf(m, cm[i]);
    m = warp_max(m);
    if (lane == 0) atomicMax(&s_max[0], __float_as_uint(m));
    __syncthreads();
    if (threadIdx.x == 0) atomicMax(absmax, s_max[0]);
  }
}

// ---- pass 2: transform, stage transposed in shared memory, quantise, store ----------------
template <typename T, int N, int ROUND>
__global__ void __launch_bounds__(kThreads) col_ht_quant_kernel(const T* __restrict__ x, ColParams p, QuantDev q,
                                                                uint8_t* __restrict__ codes, float* __restrict__ scales,
                                                                const uint32_t* __restrict__ absmax) {
  constexpr int VEC = vec_for<T, N>();
  constexpr int CPL = ColTraits<T>::kCpl;
  constexpr int CC = 32 * VEC * CPL;
  extern __shared__ __align__(16) float tile[];  // [CC][pitch]
  x += (int64_t)blockIdx.z * p.rows * p.ldx;
  codes += (int64_t)blockIdx.z * p.sample_pitch;
  const double* sawb_parts = reinterpret_cast<const double*>(absmax) + 2 * ((size_t)blockIdx.z * gridDim.y * gridDim.x);
  absmax += (size_t)blockIdx.z * (p.scale_row ? (size_t)p.cols : 1);
  scales += (size_t)blockIdx.z * (p.scale_row ? (size_t)p.cols : 1);
  // the noise / Philox element index runs on from sample to sample
  const uint64_t e_base = (uint64_t)blockIdx.z * (uint64_t)p.out_len * (uint64_t)p.cols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * CC;
  const int64_t nblk = p.rows / N;
  const int64_t blk0 = (int64_t)blockIdx.y * p.nb;
  const int r = p.r;

  constexpr int G = group_for<N>();
  for (int b = warp * G; b < p.nb; b += kWarps * G) {
    if (blk0 + b < nblk) {
      // blocks of the group past the end come back as zeros, which is what their tile slots must hold
      float v[VEC * CPL][N * G];
      load_transform<T, N, VEC>(x, p, blk0 + b, nblk, c0, lane, v);
      if constexpr (N == 1) {
        // no transform: the 16 rows of a column are 16 consecutive tile positions, stored as four float4
#pragma unroll
        for (int vv = 0; vv < VEC; ++vv)
#pragma unroll
          for (int qq = 0; qq < CPL; ++qq) {
            float4* dst = reinterpret_cast<float4*>(tile + ((lane + 32 * vv) * CPL + qq) * p.pitch + b);
            const float(&c)[G] = v[vv * CPL + qq];
#pragma unroll
            for (int g4 = 0; g4 < G / 4; ++g4) dst[g4] = make_float4(c[4 * g4], c[4 * g4 + 1], c[4 * g4 + 2], c[4 * g4 + 3]);
          }
      } else {
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const int j = p.pos[k];
          if (j >= 0) {
#pragma unroll
            for (int vv = 0; vv < VEC; ++vv)
#pragma unroll
              for (int qq = 0; qq < CPL; ++qq)
                tile[((lane + 32 * vv) * CPL + qq) * p.pitch + (b + g) * r + j] = v[vv * CPL + qq][g * N + k];
          }
        }
      }
      }
    } else {
      for (int j = 0; j < G * r; ++j)
#pragma unroll
        for (int vv = 0; vv < VEC; ++vv)
#pragma unroll
          for (int qq = 0; qq < CPL; ++qq) tile[((lane + 32 * vv) * CPL + qq) * p.pitch + b * r + j] = 0.0f;
    }
  }
  __syncthreads();

  float clip = 0.0f;  // SAWB clamp bound
  if (p.sawb) {
    // clip = 12.1 * sqrt(mean(y^2)) - 12.2 * mean(|y|) over the whole transformed tensor (of this sample)
    __shared__ double s_tot[2][kWarps];
    __shared__ float s_clip;
    const double* part = sawb_parts;
    const int nparts = (int)(gridDim.x * gridDim.y);
    double a = 0.0, b = 0.0;
    for (int i = threadIdx.x; i < nparts; i += kThreads) {
      a += part[2 * i];
      b += part[2 * i + 1];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
      b += __shfl_xor_sync(0xFFFFFFFFu, b, o);
    }
    if (lane == 0) {
      s_tot[0][warp] = a;
      s_tot[1][warp] = b;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      double ta = 0.0, tb = 0.0;
      for (int w = 0; w < kWarps; ++w) {
        ta += s_tot[0][w];
        tb += s_tot[1][w];
      }
      const double count = (double)p.out_len * (double)p.cols;
      const float rms = __fsqrt_rn((float)(ta / count));
      s_clip = __fsub_rn(__fmul_rn(12.1f, rms), __fmul_rn(12.2f, (float)(tb / count)));
    }
    __syncthreads();
    clip = s_clip;
  }
  ScalePair sp_t = scale_from_absmax(p.sawb ? clip : (p.scale_row ? 0.0f : __uint_as_float(absmax[0])), q.qmax);
  if (!p.scale_row && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) scales[0] = sp_t.s;
  const int qmax = (int)q.qmax;
  const int cpr = (p.nb * r) >> 3;  // 8-code chunks per tile row
  const int64_t pos0 = blk0 * r;    // first stored position of this tile within an output row
  // the eight codes of chunk `ch` of tile row `cl` (column c = c0 + cl); zeros past the end of the row
  auto quantise8 = [&](int cl, int ch, int (&code)[8]) {
    const int c = c0 + cl;
    const int64_t l0 = pos0 + (int64_t)ch * 8;
    if (l0 >= p.out_len) {
#pragma unroll
      for (int i = 0; i < 8; ++i) code[i] = 0;
      return;
    }
    float v[8];
    const float4 a = *reinterpret_cast<const float4*>(tile + cl * p.pitch + ch * 8);
    const float4 b = *reinterpret_cast<const float4*>(tile + cl * p.pitch + ch * 8 + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    if (p.sawb) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = fminf(fmaxf(v[i], -clip), clip);  // torch.clamp(x, -clip, clip)
    }
    ScalePair sp = sp_t;
    if (p.scale_row) {
      sp = scale_from_absmax(__uint_as_float(absmax[c]), q.qmax);
      if (blockIdx.y == 0 && ch == 0 && c < p.cols) scales[c] = sp.s;
    }
    if (ROUND == HOT_ROUND_STOCH_PHILOX) {
      // the random number of a code is indexed by its position e in the stored layout
      // batched calls index Philox by the position in the padded output row, so that runs stay aligned
      const uint64_t e0 = p.sample_pitch > 0
                              ? (uint64_t)c * (uint64_t)(p.sample_pitch * p.batch) + (uint64_t)blockIdx.z * (uint64_t)p.sample_pitch + (uint64_t)l0
                              : (uint64_t)c * (uint64_t)p.out_len + (uint64_t)l0;
      // (one block serves 16 elements with 8 random bits each, or 32 with 4 bits each)
      const int rb = rand_bits(q.qmax);
      const int shift = rb == 4 ? 5 : 4;
      if ((e0 & 7u) == 0) {
        // aligned run of 8: its random numbers are the bytes (or the low / high nibbles of the bytes) of two
        // words of one block, so they are added to the K values four at a time in packed lanes
        const uint4 blk = philox_block(q, e0 >> shift);
        uint32_t kk[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) kk[i] = philox_kbits(v[i], sp);
        uint32_t c0, c1;  // four offset codes each, one per byte
        if (rb == 4) {
          const bool hi = (e0 & 16u) != 0;
          const int nib = (int)((e0 >> 3) & 1u) * 4;
          const uint32_t r0 = ((hi ? blk.z : blk.x) >> nib) & 0x0F0F0F0Fu, r1 = ((hi ? blk.w : blk.y) >> nib) & 0x0F0F0F0Fu;
          c0 = (offset_sums4_rb4(kk[0], kk[1], kk[2], kk[3], r0) >> 4) & 0x0F0F0F0Fu;
          c1 = (offset_sums4_rb4(kk[4], kk[5], kk[6], kk[7], r1) >> 4) & 0x0F0F0F0Fu;
        } else {
          const bool hi = (e0 & 8u) != 0;
          c0 = offset_codes4_rb8(kk[0], kk[1], kk[2], kk[3], hi ? blk.z : blk.x);
          c1 = offset_codes4_rb8(kk[4], kk[5], kk[6], kk[7], hi ? blk.w : blk.y);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          code[i] = (int)((c0 >> (8 * i)) & 0xFFu) - (qmax + 1);
          code[i + 4] = (int)((c1 >> (8 * i)) & 0xFFu) - (qmax + 1);
        }
      } else {
        uint64_t g = e0 >> shift;
        uint4 blk = philox_block(q, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint64_t e = e0 + (uint64_t)i;
          if ((e >> shift) != g) {  // the run crossed into the next block (unaligned row starts only)
            g = e >> shift;
            blk = philox_block(q, g);
          }
          const uint32_t r = rb == 4 ? philox_r4(blk, e) : philox_r8(blk, e);
          code[i] = (int)philox_offset_code(v[i], sp, r, rb) - (qmax + 1);
        }
      }
    } else {
      float u[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float un = 1.0f;
        if (ROUND == HOT_ROUND_STOCH_NOISE) {
          const int64_t l = l0 + i;
          if (l < p.out_len)
            un = p.noise_transposed ? q.noise[e_base + (int64_t)c * p.out_len + l] : q.noise[e_base + l * (int64_t)p.cols + c];
        }
        u[i] = un;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) code[i] = quantise_one<ROUND>(v[i], sp, u[i], qmax);
    }
  };
  if (p.store4) {
    // packed INT4: a run of 16 codes per item; byte j = code j | code (j + 8) << 4 (nb * r is a multiple of 16)
    const int rpr = cpr >> 1;  // runs per tile row
    for (int item = threadIdx.x; item < CC * rpr; item += kThreads) {
      const int cl = item / rpr, run = item - cl * rpr;
      const int c = c0 + cl;
      const int64_t l0 = pos0 + (int64_t)run * 16;
      if (c >= p.cols || l0 >= p.out_len) continue;
      int lo[8], hi[8];
      quantise8(cl, 2 * run, lo);
      quantise8(cl, 2 * run + 1, hi);
      uint32_t w0 = 0, w1 = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w0 |= (uint32_t)((lo[i] & 0xF) | ((hi[i] & 0xF) << 4)) << (8 * i);
        w1 |= (uint32_t)((lo[i + 4] & 0xF) | ((hi[i + 4] & 0xF) << 4)) << (8 * i);
      }
      *reinterpret_cast<uint2*>(codes + (int64_t)c * p.ld_codes + (l0 >> 1)) = make_uint2(w0, w1);
    }
  } else {
    for (int item = threadIdx.x; item < CC * cpr; item += kThreads) {
      const int cl = item / cpr, ch = item - cl * cpr;
      const int c = c0 + cl;
      const int64_t l0 = pos0 + (int64_t)ch * 8;
      if (c >= p.cols || l0 >= p.out_len) continue;
      int code[8];
      quantise8(cl, ch, code);
      uint32_t w0 = 0, w1 = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w0 |= (uint32_t)(code[i] & 0xFF) << (8 * i);
        w1 |= (uint32_t)(code[i + 4] & 0xFF) << (8 * i);
      }
      *reinterpret_cast<uint2*>(codes + (int64_t)c * p.ld_codes + l0) = make_uint2(w0, w1);
    }
  }
  // batched: a sample's codes are padded with zeros up to the next sample (the GEMM contracts over them)
  if (p.sample_pitch > 0 && blk0 + p.nb >= nblk) {
    const int64_t from = (p.out_len + 7) & ~(int64_t)7;
    const int chunks = (int)((p.sample_pitch - from) >> 3);
    for (int item = threadIdx.x; item < CC * chunks; item += kThreads) {
      const int cl = item / chunks, ch = item - cl * chunks;
      if (c0 + cl < p.cols) *reinterpret_cast<uint2*>(codes + (int64_t)(c0 + cl) * p.ld_codes + from + ch * 8) = make_uint2(0u, 0u);
    }
  }
}

// ---- un-quantised projection and its transpose (schemes that quantise the projected tensor in its
// natural layout, or expand a low-rank gradient back to all tokens) --------------------------------
// out[(b * r + j), c] = sum_t H_N[sel[j], t] * x[b * N + t, c], float32, same butterfly as above
template <typename T, int N>
__global__ void __launch_bounds__(kThreads) hla_project_kernel(const T* __restrict__ x, ColParams p, float* __restrict__ out,
                                                               int64_t ldo) {
  constexpr int VEC = vec_for<T, N>();
  constexpr int CPL = ColTraits<T>::kCpl;
  constexpr int CC = 32 * VEC * CPL;
  constexpr int G = group_for<N>();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * CC;
  const int64_t nblk = p.rows / N;
  const int64_t blk0 = (int64_t)blockIdx.y * p.nb;
  for (int b = warp * G; b < p.nb; b += kWarps * G) {
    if (blk0 + b >= nblk) break;
    float v[VEC * CPL][N * G];
    load_transform<T, N, VEC>(x, p, blk0 + b, nblk, c0, lane, v);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (blk0 + b + g >= nblk) break;
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const int j = p.pos[k];
        if (j < 0) continue;
        float* row = out + ((blk0 + b + g) * p.r + j) * ldo;
#pragma unroll
        for (int vv = 0; vv < VEC; ++vv)
#pragma unroll
          for (int qq = 0; qq < CPL; ++qq) {
            const int c = c0 + (lane + 32 * vv) * CPL + qq;
            if (c < p.cols) row[c] = v[vv * CPL + qq][g * N + k];
          }
      }
    }
  }
}

// out[b * N + t, c] = scale * sum_j H_N[sel[j], t] * in[b * r + j, c]: the kept rows go back to their
// places in a zero block and the (symmetric) butterfly runs over it, in the same fixed order
template <typename TO, int N>
__global__ void __launch_bounds__(kThreads) hla_expand_kernel(const float* __restrict__ in, int64_t ldi, ColParams p, float scale,
                                                              TO* __restrict__ out, int64_t ldo) {
  const int c = blockIdx.x * kThreads + threadIdx.x;
  if (c >= p.cols) return;
  const int64_t nblk = p.rows / N;
  for (int64_t blk = blockIdx.y; blk < nblk; blk += gridDim.y) {
    float v[N];
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const int j = p.pos[k];
      v[k] = j >= 0 ? in[(blk * p.r + j) * ldi + c] : 0.0f;
    }
    butterfly_regs<N, 0, N>(v);
#pragma unroll
    for (int t = 0; t < N; ++t) {
      const float y = __fmul_rn(v[t], scale);
      if (sizeof(TO) == 2) reinterpret_cast<__nv_bfloat16*>(out)[(blk * N + t) * ldo + c] = __float2bfloat16_rn(y);
      else reinterpret_cast<float*>(out)[(blk * N + t) * ldo + c] = y;
    }
  }
}

template <typename T, int N>
int launch_n(const T* x, const ColParams& p, const hot_quant_t& hq, uint8_t* codes, float* scales, uint32_t* ws,
             cudaStream_t st) {
  constexpr int VEC = vec_for<T, N>();
  constexpr int CC = 32 * VEC * ColTraits<T>::kCpl;
  const QuantDev q = make_quant_dev(hq);
  const int64_t nblk = p.rows / N;
  dim3 grid((unsigned)((p.cols + CC - 1) / CC), (unsigned)((nblk + p.nb - 1) / p.nb), (unsigned)p.batch);
  const size_t smem = (size_t)CC * p.pitch * sizeof(float);
  if (!p.sawb) HOT_CUDA(cudaMemsetAsync(ws, 0, sizeof(uint32_t) * (p.scale_row ? (size_t)p.cols * p.batch : (size_t)p.batch), st));
  col_ht_absmax_kernel<T, N><<<grid, kThreads, 0, st>>>(x, p, ws);
  auto launch = [&](auto kernel) -> int {
    HOT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kThreads, smem, st>>>(x, p, q, codes, scales, ws);
    return HOT_OK;
  };
  int rc;
  switch (hq.rounding) {
    case HOT_ROUND_NEAREST: rc = launch(col_ht_quant_kernel<T, N, HOT_ROUND_NEAREST>); break;
    case HOT_ROUND_STOCH_PHILOX: rc = launch(col_ht_quant_kernel<T, N, HOT_ROUND_STOCH_PHILOX>); break;
    default: rc = launch(col_ht_quant_kernel<T, N, HOT_ROUND_STOCH_NOISE>); break;
  }
  if (rc) return rc;
  HOT_CUDA(cudaGetLastError());
  return HOT_OK;
}

template <typename T>
int launch_t(const T* x, int n, const ColParams& p, const hot_quant_t& hq, uint8_t* codes, float* scales, uint32_t* ws,
             cudaStream_t st) {
  switch (n) {
    case 1: return launch_n<T, 1>(x, p, hq, codes, scales, ws, st);
    case 2: return launch_n<T, 2>(x, p, hq, codes, scales, ws, st);
    case 4: return launch_n<T, 4>(x, p, hq, codes, scales, ws, st);
    case 8: return launch_n<T, 8>(x, p, hq, codes, scales, ws, st);
    case 16: return launch_n<T, 16>(x, p, hq, codes, scales, ws, st);
    case 32: return launch_n<T, 32>(x, p, hq, codes, scales, ws, st);
    case 64: return launch_n<T, 64>(x, p, hq, codes, scales, ws, st);
  }
  HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_col_ht_quant: order %d not in {1,2,4,8,16,32,64}", n);
}

}  // namespace
}  // namespace hot

namespace hot {
namespace {
// tile geometry shared by the launcher and the scratch-size query
void col_tile_geometry(int dtype, int order, int r, int* cc, int* nb) {
  const int cpl = dtype == HOT_BF16 ? 2 : 1;
  const int per = 64 / ((order < 16 ? 16 : order) * cpl);
  const int vec = per >= 4 ? 4 : (per >= 2 ? 2 : 1);
  *cc = 32 * vec * cpl;
  // the smaller of the two tile heights the launcher may use (INT8 / packed INT4 output): an upper bound on CTAs
  int b8 = (128 / r) / 8 * 8, b16 = (128 / r) / 16 * 16;
  if (b8 < 8) b8 = 8;
  if (b16 < 16) b16 = 16;
  *nb = b8 < b16 ? b8 : b16;
}
}  // namespace
}  // namespace hot

extern "C" size_t hot_col_ht_quant_scratch_words(int dtype, int64_t rows, int64_t cols, int order, int r, int scale_mode) {
  if (rows < 0 || cols <= 0 || order < 1 || r < 1 || r > order) return 0;
  if (scale_mode == HOT_SCALE_TENSOR) return 1;
  if (scale_mode == HOT_SCALE_ROW) return (size_t)cols;
  int cc, nb;
  hot::col_tile_geometry(dtype, order, r, &cc, &nb);
  const int64_t nblk = rows / order;
  return 4 * (size_t)((cols + cc - 1) / cc) * (size_t)((nblk + nb - 1) / nb) + 4;  // two doubles per CTA
}

namespace hot {
namespace {
// batch > 1: x holds `batch` samples of `rows` rows each; sample b's codes start sample_pitch * b bytes into each output row
int col_ht_quant_impl(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order, const int32_t* sel, int r,
                      const hot_quant_t* q, int logical_layout, void* codes_t, int64_t ld_codes, float* scales,
                      uint32_t* absmax_ws, hot_stream_t stream, int batch, int64_t sample_pitch) {
  if (!x || !q || !codes_t || !scales || !sel || !absmax_ws) HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant: null pointer");
  if (rows < 0 || cols <= 0 || cols > (1 << 30)) HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant: bad shape");
  if (int rc = validate_quant(q, "hot_col_ht_quant")) return rc;
  if (order < 1 || order > 64 || (order & (order - 1)))
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_col_ht_quant: order %d not a power of two in [1, 64]", order);
  if (rows % order != 0) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_col_ht_quant: rows %lld not a multiple of order %d", (long long)rows, order);
  if (r < 1 || r > order) HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant: rank %d outside [1, %d]", r, order);
  const int esz = dtype == HOT_F32 ? 4 : 2;
  if (dtype != HOT_F32 && dtype != HOT_BF16) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_col_ht_quant: dtype %d", dtype);
  if (ldx < cols || (ldx * esz) % 4 != 0 || ((uintptr_t)x) % 4 != 0 || (dtype == HOT_BF16 && cols % 2 != 0))
    HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant: x pitch must be >= cols and 4-byte aligned (bf16: even cols)");
  ColParams p;
  p.rows = rows;
  p.cols = (int)cols;
  p.ldx = ldx;
  p.ld_codes = ld_codes;
  p.r = r;
  p.out_len = rows / order * r;
  p.scale_row = q->scale_mode == HOT_SCALE_ROW;
  p.sawb = q->scale_mode == HOT_SCALE_SAWB;
  if (p.sawb && q->rounding != HOT_ROUND_NEAREST)
    HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant: HOT_SCALE_SAWB goes with HOT_ROUND_NEAREST (the reference's sawb_quantizer rounds to nearest)");
  if (p.sawb && ((uintptr_t)absmax_ws) % 8 != 0) HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant: scratch must be 8-byte aligned for HOT_SCALE_SAWB");
  p.store4 = q->storage == HOT_STORE_INT4;
  p.noise_transposed = logical_layout == HOT_LAYOUT_TRANSPOSED;
  p.batch = batch;
  p.sample_pitch = sample_pitch;
  for (int k = 0; k < 64; ++k) p.pos[k] = -1;
  for (int j = 0; j < r; ++j) {
    if (sel[j] < 0 || sel[j] >= order || p.pos[sel[j]] >= 0)
      HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant: sel[%d] = %d out of range or repeated", j, sel[j]);
    p.pos[sel[j]] = (signed char)j;
  }
  // blocks per tile: a multiple of 8 (so that nb * r is a multiple of 8 codes) near 128 / r
  // (packed INT4 output: a multiple of 16, so that nb * r is whole runs of 16 codes)
  const int step = p.store4 ? 16 : 8;
  int nb = (128 / r) / step * step;
  if (nb < step) nb = step;
  p.nb = nb;
  p.pitch = ((nb * r + 31) / 32) * 32 + 4;
  const int64_t row_bytes = p.store4 ? (p.out_len + 1) / 2 : p.out_len;
  if (sample_pitch > 0) {
    if (p.store4) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_col_ht_quant_batched: HOT_STORE_INT8 only");
    if (sample_pitch % 16 != 0 || sample_pitch < ((row_bytes + 7) / 8) * 8 || ld_codes < sample_pitch * batch)
      HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant_batched: sample pitch %lld must be a multiple of 16, >= %lld, and fit the row pitch",
               (long long)sample_pitch, (long long)row_bytes);
  }
  if (ld_codes % 16 != 0 || ld_codes < ((row_bytes + 7) / 8) * 8 || ((uintptr_t)codes_t) % 16 != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant: codes pitch %lld must be a multiple of 16 and >= %lld", (long long)ld_codes,
             (long long)row_bytes);
  if (rows == 0) return HOT_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HOT_F32) return launch_t<float>((const float*)x, order, p, *q, (uint8_t*)codes_t, scales, absmax_ws, st);
  return launch_t<__nv_bfloat16>((const __nv_bfloat16*)x, order, p, *q, (uint8_t*)codes_t, scales, absmax_ws, st);
}
}  // namespace
}  // namespace hot

extern "C" int hot_col_ht_quant(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order,
                                const int32_t* sel, int r, const hot_quant_t* q, int logical_layout, void* codes_t,
                                int64_t ld_codes, float* scales, uint32_t* absmax_ws, hot_stream_t stream) {
  return hot::col_ht_quant_impl(x, dtype, rows, cols, ldx, order, sel, r, q, logical_layout, codes_t, ld_codes, scales,
                                absmax_ws, stream, 1, 0);
}

extern "C" int hot_col_ht_quant_batched(const void* x, int dtype, int64_t batch, int64_t rows, int64_t cols, int64_t ldx,
                                        int order, const int32_t* sel, int r, const hot_quant_t* q, int logical_layout,
                                        void* codes_t, int64_t ld_codes, int64_t sample_pitch, float* scales,
                                        uint32_t* absmax_ws, hot_stream_t stream) {
  using namespace hot;
  if (batch < 1 || batch > 65535) HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant_batched: batch %lld outside [1, 65535]", (long long)batch);
  if (sample_pitch <= 0) HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant_batched: sample pitch must be positive");
  return col_ht_quant_impl(x, dtype, rows, cols, ldx, order, sel, r, q, logical_layout, codes_t, ld_codes, scales,
                           absmax_ws, stream, (int)batch, sample_pitch);
}

// ---------------------------------------------------------------------------------------
// Variant for callers that cannot hand over scratch memory of their own.
// ---------------------------------------------------------------------------------------
namespace hot {
namespace {

constexpr int kStaticScratchWords = 16384;  // 64 KiB, resident on every GPU that loads this library

// The abs-max words of hot_col_ht_quant_static live here instead of in a caller buffer.  In host
// code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) uint32_t g_static_scratch[kStaticScratchWords];

uint32_t* g_static_scratch_ptr[kMaxDevices] = {};  // device address per device ordinal, filled on first use

// Device address of g_static_scratch on the CURRENT device.  The first call on a device asks
// the runtime for it (which may load the module: not something to do under stream capture).
int static_scratch_for_current_device(uint32_t** out) {
  int dev = -1;
  HOT_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_col_ht_quant_static: device ordinal %d", dev);
  uint32_t* p = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void* sym = nullptr;
    HOT_CUDA(cudaGetSymbolAddress(&sym, g_static_scratch));
    if (!sym) HOT_FAIL(HOT_ERR_CUDA, "hot_col_ht_quant_static: cudaGetSymbolAddress returned a null address");
    p = static_cast<uint32_t*>(sym);
    __atomic_store_n(&g_static_scratch_ptr[dev], p, __ATOMIC_RELEASE);  // racing first calls store the same value
  }
  *out = p;
  return HOT_OK;
}

}  // namespace
}  // namespace hot

extern "C" int hot_col_ht_quant_static(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order,
                                       const int32_t* sel, int r, const hot_quant_t* q, int logical_layout,
                                       void* codes_t, int64_t ld_codes, float* scales, hot_stream_t stream) {
  using namespace hot;
  if (!q) HOT_FAIL(HOT_ERR_ARG, "hot_col_ht_quant_static: null pointer");
  const int64_t words = (int64_t)hot_col_ht_quant_scratch_words(dtype, rows, cols, order, r, q->scale_mode);
  if (words > kStaticScratchWords)
    HOT_FAIL(HOT_ERR_UNSUPPORTED,
             "hot_col_ht_quant_static: this scale mode over %lld columns needs %lld scratch words, the built-in scratch "
             "holds %d; use hot_col_ht_quant with a caller-owned scratch buffer",
             (long long)cols, (long long)words, kStaticScratchWords);
  uint32_t* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  // What the previous call left in the array does not leak into this one: in the abs-max modes
  // (HOT_SCALE_TENSOR, HOT_SCALE_ROW) hot_col_ht_quant zeroes the words it uses with a memset on
  // the stream before its first kernel; in HOT_SCALE_SAWB mode there is no memset, and every CTA
  // of the statistics kernel overwrites its own four words before the second kernel reads them
  return hot_col_ht_quant(x, dtype, rows, cols, ldx, order, sel, r, q, logical_layout, codes_t, ld_codes, scales, scratch,
                          stream);
}

// ---------------------------------------------------------------------------------------
// Un-quantised low-rank projection along the first dim, and its transpose.
// ---------------------------------------------------------------------------------------
namespace hot {
namespace {
int fill_selection(ColParams& p, int order, const int32_t* sel, int r, const char* who) {
  if (order < 1 || order > 64 || (order & (order - 1))) HOT_FAIL(HOT_ERR_UNSUPPORTED, "%s: order %d not a power of two in [1, 64]", who, order);
  if (!sel || r < 1 || r > order) HOT_FAIL(HOT_ERR_ARG, "%s: rank %d outside [1, %d] or null selection", who, r, order);
  for (int k = 0; k < 64; ++k) p.pos[k] = -1;
  for (int j = 0; j < r; ++j) {
    if (sel[j] < 0 || sel[j] >= order || p.pos[sel[j]] >= 0) HOT_FAIL(HOT_ERR_ARG, "%s: sel[%d] = %d out of range or repeated", who, j, sel[j]);
    p.pos[sel[j]] = (signed char)j;
  }
  p.r = r;
  return HOT_OK;
}

template <typename T, int N>
int project_n(const T* x, const ColParams& p, float* out, int64_t ldo, cudaStream_t st) {
  constexpr int CC = 32 * vec_for<T, N>() * ColTraits<T>::kCpl;
  const int64_t nblk = p.rows / N;
  dim3 grid((unsigned)((p.cols + CC - 1) / CC), (unsigned)((nblk + p.nb - 1) / p.nb));
  hla_project_kernel<T, N><<<grid, kThreads, 0, st>>>(x, p, out, ldo);
  HOT_CUDA(cudaGetLastError());
  return HOT_OK;
}
template <typename T>
int project_t(const T* x, int n, const ColParams& p, float* out, int64_t ldo, cudaStream_t st) {
  switch (n) {
    case 1: return project_n<T, 1>(x, p, out, ldo, st);
    case 2: return project_n<T, 2>(x, p, out, ldo, st);
    case 4: return project_n<T, 4>(x, p, out, ldo, st);
    case 8: return project_n<T, 8>(x, p, out, ldo, st);
    case 16: return project_n<T, 16>(x, p, out, ldo, st);
    case 32: return project_n<T, 32>(x, p, out, ldo, st);
    default: return project_n<T, 64>(x, p, out, ldo, st);
  }
}
template <typename TO, int N>
int expand_n(const float* in, int64_t ldi, const ColParams& p, float scale, TO* out, int64_t ldo, cudaStream_t st) {
  const int64_t nblk = p.rows / N;
  dim3 grid((unsigned)((p.cols + kThreads - 1) / kThreads), (unsigned)(nblk < 4096 ? nblk : 4096));
  hla_expand_kernel<TO, N><<<grid, kThreads, 0, st>>>(in, ldi, p, scale, out, ldo);
  HOT_CUDA(cudaGetLastError());
  return HOT_OK;
}
template <typename TO>
int expand_t(const float* in, int64_t ldi, int n, const ColParams& p, float scale, TO* out, int64_t ldo, cudaStream_t st) {
  switch (n) {
    case 1: return expand_n<TO, 1>(in, ldi, p, scale, out, ldo, st);
    case 2: return expand_n<TO, 2>(in, ldi, p, scale, out, ldo, st);
    case 4: return expand_n<TO, 4>(in, ldi, p, scale, out, ldo, st);
    case 8: return expand_n<TO, 8>(in, ldi, p, scale, out, ldo, st);
    case 16: return expand_n<TO, 16>(in, ldi, p, scale, out, ldo, st);
    case 32: return expand_n<TO, 32>(in, ldi, p, scale, out, ldo, st);
    default: return expand_n<TO, 64>(in, ldi, p, scale, out, ldo, st);
  }
}
}  // namespace
}  // namespace hot

extern "C" int hot_hla_project(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order, const int32_t* sel,
                               int r, float* out, int64_t ldo, hot_stream_t stream) {
  using namespace hot;
  if (!x || !out) HOT_FAIL(HOT_ERR_ARG, "hot_hla_project: null pointer");
  if (rows < 0 || cols <= 0 || cols > (1 << 30)) HOT_FAIL(HOT_ERR_ARG, "hot_hla_project: bad shape");
  if (dtype != HOT_F32 && dtype != HOT_BF16) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_hla_project: dtype %d", dtype);
  ColParams p = {};
  if (int rc = fill_selection(p, order, sel, r, "hot_hla_project")) return rc;
  if (rows % order != 0) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_hla_project: rows %lld not a multiple of order %d", (long long)rows, order);
  const int esz = dtype == HOT_F32 ? 4 : 2;
  if (ldx < cols || (ldx * esz) % 4 != 0 || ((uintptr_t)x) % 4 != 0 || (dtype == HOT_BF16 && cols % 2 != 0) || ldo < cols)
    HOT_FAIL(HOT_ERR_ARG, "hot_hla_project: pitches must cover cols; x 4-byte aligned (bf16: even cols)");
  p.rows = rows;
  p.cols = (int)cols;
  p.ldx = ldx;
  p.nb = 64;
  p.batch = 1;
  if (rows == 0) return HOT_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HOT_F32) return project_t<float>((const float*)x, order, p, out, ldo, st);
  return project_t<__nv_bfloat16>((const __nv_bfloat16*)x, order, p, out, ldo, st);
}

extern "C" int hot_hla_expand(const float* in, int64_t ldi, int64_t rows_out, int64_t cols, int order, const int32_t* sel, int r,
                              float scale, void* out, int out_dtype, int64_t ldo, hot_stream_t stream) {
  using namespace hot;
  if (!in || !out) HOT_FAIL(HOT_ERR_ARG, "hot_hla_expand: null pointer");
  if (rows_out < 0 || cols <= 0 || cols > (1 << 30) || ldi < cols || ldo < cols) HOT_FAIL(HOT_ERR_ARG, "hot_hla_expand: bad shape or pitch");
  if (out_dtype != HOT_F32 && out_dtype != HOT_BF16) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_hla_expand: out dtype %d", out_dtype);
  ColParams p = {};
  if (int rc = fill_selection(p, order, sel, r, "hot_hla_expand")) return rc;
  if (rows_out % order != 0) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_hla_expand: rows %lld not a multiple of order %d", (long long)rows_out, order);
  p.rows = rows_out;
  p.cols = (int)cols;
  if (rows_out == 0) return HOT_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dtype == HOT_F32) return expand_t<float>(in, ldi, order, p, scale, (float*)out, ldo, st);
  return expand_t<__nv_bfloat16>(in, ldi, order, p, scale, (__nv_bfloat16*)out, ldo, st);
}
