// Fused block-Hadamard transform along the contiguous dim + INT4/INT8 quantisation.
//
// Data layout: every thread owns vectors of 8 consecutive elements (two 128-bit loads for
// fp32, one for bf16).  Butterfly stages h = 1, 2, 4 run inside the thread; stages
// h = 8, 16, 32 exchange with lane ^ (h / 8) through warp shuffles, so a Hadamard block of
// order n <= 64 lives in n / 8 adjacent lanes.  The arithmetic per stage is (x + y, x - y)
// on the pair (i, i + h), the order the CPU oracle fixes.
//
// Per-row ("per-token") scale: one launch; a row is held in registers by `tpr` threads,
// reduced to its abs-max, then quantised and stored.
// Per-tensor scale: two launches over the same input (abs-max into a scratch word, then
// quantise); both are pure streaming loops.
#include "common.cuh"

namespace hot {
namespace {

constexpr int kThreads = 256;
constexpr int kVmax = 8;  // vectors per thread in the per-row kernel: cols <= 8 * 8 * 256

__device__ __forceinline__ void butterfly8(float (&v)[8], int n) {
  if (n >= 2) {
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const float a = v[i], b = v[i + 1];
      v[i] = a + b;
      v[i + 1] = a - b;
    }
  }
  if (n >= 4) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & 2) == 0) {
        const float a = v[i], b = v[i + 2];
        v[i] = a + b;
        v[i + 2] = a - b;
      }
    }
  }
  if (n >= 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = v[i], b = v[i + 4];
      v[i] = a + b;
      v[i + 4] = a - b;
    }
  }
}

// Stages h = 8 .. n/2 across lanes.  Must be executed by all 32 lanes.
__device__ __forceinline__ void butterfly_lanes(float (&v)[8], int n, int lane) {
  for (int h = 8; h < n; h <<= 1) {
    const int m = h >> 3;
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float o = __shfl_xor_sync(0xFFFFFFFFu, v[i], m);
      v[i] = upper ? (o - v[i]) : (v[i] + o);
    }
  }
}

__device__ __forceinline__ float absmax8(const float (&v)[8]) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
  return m;
}

// Quantise 8 transformed values whose first logical element index is `e0` (a multiple of 8)
// and store them at `dst` (already offset to the vector).
template <int ROUND, int STORE4>
__device__ __forceinline__ void quantise_store8(const float (&v)[8], const ScalePair& sp, const QuantDev& q, uint64_t e0,
                                                uint8_t* dst) {
  float u[8];
  uint32_t r16[8];
  if (ROUND == HOT_ROUND_STOCH_PHILOX) philox_bits8(q, e0 >> 3, r16);
  if (ROUND == HOT_ROUND_STOCH_NOISE) Load8<float>::run(q.noise + e0, u);
  const int qmax = (int)q.qmax;
  int c[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    c[i] = quantise_one<ROUND>(v[i], sp, ROUND == HOT_ROUND_STOCH_NOISE ? u[i] : 0.0f,
                               ROUND == HOT_ROUND_STOCH_PHILOX ? r16[i] : 0u, qmax);
  if (STORE4) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) w |= (uint32_t)(c[i] & 0xF) << (4 * i);
    *reinterpret_cast<uint32_t*>(dst) = w;
  } else {
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w0 |= (uint32_t)(c[i] & 0xFF) << (8 * i);
      w1 |= (uint32_t)(c[i + 4] & 0xFF) << (8 * i);
    }
    *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
  }
}

// ---------------------------------------------------------------------------------------
// per-row scale: one pass, row resident in registers
// ---------------------------------------------------------------------------------------
template <typename T, int ROUND, int STORE4>
__global__ void __launch_bounds__(kThreads) row_ht_quant_rowscale_kernel(
    const T* __restrict__ x, int64_t rows, int cols, int64_t ldx, int n, QuantDev q, uint8_t* __restrict__ codes,
    int64_t ld_codes, float* __restrict__ scales, int tpr) {
  __shared__ float s_part[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rows_per_cta = kThreads / tpr;
  const int64_t row = (int64_t)blockIdx.x * rows_per_cta + threadIdx.x / tpr;
  const int t = threadIdx.x % tpr;
  const int nvec = cols >> 3;
  const int nv = (nvec + tpr - 1) / tpr;  // uniform over the CTA
  const bool row_ok = row < rows;
  const T* xr = x + (row_ok ? row : 0) * ldx;

  float v[kVmax][8];
  float mx = 0.0f;
#pragma unroll
  for (int j = 0; j < kVmax; ++j) {
    if (j < nv) {
      const int vi = t + j * tpr;
      if (row_ok && vi < nvec) {
        Load8<T>::run(xr + (int64_t)vi * 8, v[j]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j][i] = 0.0f;
      }
      butterfly8(v[j], n);
      butterfly_lanes(v[j], n, lane);
      mx = fmaxf(mx, absmax8(v[j]));
    }
  }
  mx = warp_max(mx);
  if (tpr > 32) {
    if (lane == 0) s_part[warp] = mx;
    __syncthreads();
    const int w0 = (threadIdx.x / tpr) * (tpr / 32);
    mx = 0.0f;
    for (int w = 0; w < tpr / 32; ++w) mx = fmaxf(mx, s_part[w0 + w]);
  }
  const ScalePair sp = scale_from_absmax(mx, q.qmax);
  if (row_ok && t == 0) scales[row] = sp.s;
  if (!row_ok) return;
  uint8_t* cr = codes + row * ld_codes;
#pragma unroll
  for (int j = 0; j < kVmax; ++j) {
    if (j < nv) {
      const int vi = t + j * tpr;
      if (vi < nvec) {
        const uint64_t e0 = (uint64_t)row * (uint64_t)cols + (uint64_t)vi * 8u;
        quantise_store8<ROUND, STORE4>(v[j], sp, q, e0, cr + (int64_t)vi * (STORE4 ? 4 : 8));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// per-tensor scale: pass 1 (abs-max) and pass 2 (quantise), streaming over vectors
// ---------------------------------------------------------------------------------------
constexpr int kUnroll = 4;

// Where vector `item` (row-major over rows x nvec) lives.  CONTIG: pitch == cols, so the tensor is
// one flat run of vectors and no division is needed.
template <bool CONTIG>
__device__ __forceinline__ void locate(int64_t item, int nvec, int64_t ldx, int64_t ld_codes, int code_bytes,
                                       int64_t& x_off, int64_t& c_off) {
  if (CONTIG) {
    x_off = item * 8;
    c_off = item * code_bytes;
  } else {
    const int64_t row = item / nvec;
    const int vi = (int)(item - row * nvec);
    x_off = row * ldx + (int64_t)vi * 8;
    c_off = row * ld_codes + (int64_t)vi * code_bytes;
  }
}

template <typename T, bool CONTIG>
__global__ void __launch_bounds__(kThreads) row_ht_absmax_kernel(const T* __restrict__ x, int64_t rows, int cols,
                                                                 int64_t ldx, int n, uint32_t* __restrict__ absmax) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const int64_t total = rows * nvec;
  const int64_t warp_id = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  float mx = 0.0f;
  for (int64_t base = warp_id * (32 * kUnroll); base < total; base += nwarps * (32 * kUnroll)) {
    float v[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t item = base + u * 32 + lane;
      if (item < total) {
        int64_t xo, co;
        locate<CONTIG>(item, nvec, ldx, 0, 0, xo, co);
        Load8<T>::run(x + xo, v[u]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      butterfly8(v[u], n);
      butterfly_lanes(v[u], n, lane);
      mx = fmaxf(mx, absmax8(v[u]));
    }
  }
  mx = warp_max(mx);
  if (lane == 0) atomic_absmax(absmax, mx);
}

template <typename T, int ROUND, int STORE4, bool CONTIG>
__global__ void __launch_bounds__(kThreads) row_ht_quant_tensorscale_kernel(
    const T* __restrict__ x, int64_t rows, int cols, int64_t ldx, int n, QuantDev q, uint8_t* __restrict__ codes,
    int64_t ld_codes, float* __restrict__ scales, const uint32_t* __restrict__ absmax) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const int64_t total = rows * nvec;
  const int64_t warp_id = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const ScalePair sp = scale_from_absmax(__uint_as_float(*absmax), q.qmax);
  if (blockIdx.x == 0 && threadIdx.x == 0) scales[0] = sp.s;
  for (int64_t base = warp_id * (32 * kUnroll); base < total; base += nwarps * (32 * kUnroll)) {
    float v[kUnroll][8];
    int64_t coff[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t item = base + u * 32 + lane;
      coff[u] = -1;
      if (item < total) {
        int64_t xo;
        locate<CONTIG>(item, nvec, ldx, ld_codes, STORE4 ? 4 : 8, xo, coff[u]);
        Load8<T>::run(x + xo, v[u]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      butterfly8(v[u], n);
      butterfly_lanes(v[u], n, lane);
      // logical element index of the vector: row * cols + col == item * 8 in either layout
      if (coff[u] >= 0) quantise_store8<ROUND, STORE4>(v[u], sp, q, (uint64_t)(base + u * 32 + lane) * 8u, codes + coff[u]);
    }
  }
}

int grid_for(int64_t total_vec, int device_sms) {
  const int64_t per_cta = (int64_t)kThreads * kUnroll;
  int64_t want = (total_vec + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)device_sms * 8;  // 8 resident CTAs of 256 threads per SM
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}

template <typename T, int ROUND, int STORE4>
int launch_typed(const T* x, int64_t rows, int cols, int64_t ldx, int n, const hot_quant_t& hq, uint8_t* codes,
                 int64_t ld_codes, float* scales, uint32_t* absmax_ws, cudaStream_t st, int sms) {
  const QuantDev q = make_quant_dev(hq);
  if (hq.scale_mode == HOT_SCALE_ROW) {
    const int nvec = cols >> 3;
    int tpr = 32;
    while (tpr < kThreads && (nvec + tpr - 1) / tpr > kVmax) tpr <<= 1;
    if ((nvec + tpr - 1) / tpr > kVmax)
      HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant: per-row scale supports cols <= %d (got %d)",
               kVmax * 8 * kThreads, cols);
    const int rows_per_cta = kThreads / tpr;
    const int64_t grid = (rows + rows_per_cta - 1) / rows_per_cta;
    row_ht_quant_rowscale_kernel<T, ROUND, STORE4>
        <<<(unsigned)grid, kThreads, 0, st>>>(x, rows, cols, ldx, n, q, codes, ld_codes, scales, tpr);
  } else {
    const int grid = grid_for(rows * (cols >> 3), sms);
    HOT_CUDA(cudaMemsetAsync(absmax_ws, 0, sizeof(uint32_t), st));
    const bool contig = ldx == cols && ld_codes == (STORE4 ? cols / 2 : cols);
    if (contig) {
      row_ht_absmax_kernel<T, true><<<grid, kThreads, 0, st>>>(x, rows, cols, ldx, n, absmax_ws);
      row_ht_quant_tensorscale_kernel<T, ROUND, STORE4, true>
          <<<grid, kThreads, 0, st>>>(x, rows, cols, ldx, n, q, codes, ld_codes, scales, absmax_ws);
    } else {
      row_ht_absmax_kernel<T, false><<<grid, kThreads, 0, st>>>(x, rows, cols, ldx, n, absmax_ws);
      row_ht_quant_tensorscale_kernel<T, ROUND, STORE4, false>
          <<<grid, kThreads, 0, st>>>(x, rows, cols, ldx, n, q, codes, ld_codes, scales, absmax_ws);
    }
  }
  HOT_CUDA(cudaGetLastError());
  return HOT_OK;
}

template <typename T>
int launch_modes(const T* x, int64_t rows, int cols, int64_t ldx, int n, const hot_quant_t& q, uint8_t* codes,
                 int64_t ld_codes, float* scales, uint32_t* ws, cudaStream_t st, int sms) {
#define HOT_CASE(R, S)                                                                              \
  if (q.rounding == (R) && q.storage == (S))                                                        \
    return launch_typed<T, (R), (S)>(x, rows, cols, ldx, n, q, codes, ld_codes, scales, ws, st, sms);
  HOT_CASE(HOT_ROUND_NEAREST, HOT_STORE_INT8)
  HOT_CASE(HOT_ROUND_NEAREST, HOT_STORE_INT4)
  HOT_CASE(HOT_ROUND_STOCH_PHILOX, HOT_STORE_INT8)
  HOT_CASE(HOT_ROUND_STOCH_PHILOX, HOT_STORE_INT4)
  HOT_CASE(HOT_ROUND_STOCH_NOISE, HOT_STORE_INT8)
  HOT_CASE(HOT_ROUND_STOCH_NOISE, HOT_STORE_INT4)
#undef HOT_CASE
  HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: bad rounding/storage %d/%d", q.rounding, q.storage);
}

}  // namespace

int device_sm_count();

}  // namespace hot

extern "C" int hot_row_ht_quant(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order,
                                const hot_quant_t* q, void* codes, int64_t ld_codes, float* scales,
                                uint32_t* absmax_ws, hot_stream_t stream) {
  using namespace hot;
  if (rows == 0 && cols > 0 && q) return HOT_OK;  // nothing to do (and the pointers may be null)
  if (!x || !q || !codes || !scales) HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: null pointer");
  if (rows < 0 || cols <= 0) HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: bad shape %lld x %lld", (long long)rows, (long long)cols);
  if (int rc = validate_quant(q, "hot_row_ht_quant")) return rc;
  if (order < 1 || order > 64 || (order & (order - 1)))
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant: order %d not a power of two in [1, 64]", order);
  if (cols % 8 != 0 || cols % order != 0 || cols > (1 << 30))
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant: cols %lld must be a multiple of 8 and of the order %d",
             (long long)cols, order);
  const int esz = dtype == HOT_F32 ? 4 : 2;
  if (ldx < cols || (ldx * esz) % 16 != 0 || ((uintptr_t)x) % 16 != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: x and its pitch must be 16-byte aligned, ldx >= cols");
  const int64_t row_bytes = q->storage == HOT_STORE_INT4 ? cols / 2 : cols;
  if (ld_codes < row_bytes || ld_codes % 8 != 0 || ((uintptr_t)codes) % 8 != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: codes pitch %lld must be >= %lld and 8-byte aligned", (long long)ld_codes,
             (long long)row_bytes);
  if (q->scale_mode == HOT_SCALE_TENSOR && !absmax_ws) HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: absmax_ws is null");
  if (q->rounding == HOT_ROUND_STOCH_NOISE && ((uintptr_t)q->noise) % 16 != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: noise must be 16-byte aligned");
  if (rows == 0) return HOT_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int sms = device_sm_count();
  if (sms <= 0) return HOT_ERR_CUDA;
  if (dtype == HOT_F32)
    return launch_modes<float>((const float*)x, rows, (int)cols, ldx, order, *q, (uint8_t*)codes, ld_codes, scales,
                               absmax_ws, st, sms);
  if (dtype == HOT_BF16)
    return launch_modes<__nv_bfloat16>((const __nv_bfloat16*)x, rows, (int)cols, ldx, order, *q, (uint8_t*)codes,
                                       ld_codes, scales, absmax_ws, st, sms);
  HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant: dtype %d", dtype);
}
