// Fused block-Hadamard transform along the contiguous dim + INT4/INT8 quantisation.
//
// Data layout: every thread owns runs of 16 consecutive elements, loaded with 128-bit loads as
// two 8-element halves A and B and held as eight packed pairs (A_i, B_i).  Blackwell's packed
// fp32 instructions (add/fma .f32x2, IEEE round-to-nearest per lane) then run the butterfly
// stages h = 1, 2, 4 of both halves at once; stage h = 8 combines A_i with B_i; stages h = 16
// and 32 exchange with lane ^ 1 and lane ^ 2 through warp shuffles.  Per stage the arithmetic
// is (x + y, x - y) on the pair (i, i + h): the order the CPU oracle fixes.  The division by
// the scale and the rounding run packed as well.
//
// Per-row ("per-token") scale: one launch; a row is held in registers by `tpr` threads,
// reduced to its abs-max, then quantised and stored.
// Per-tensor scale: two launches over the same input (abs-max into a scratch word, then
// quantise); both are pure streaming loops.
#include "ht_device.cuh"

namespace hot {
namespace {

constexpr int kThreads = 256;
constexpr int kVmaxLimit = 4;  // 16-element runs per thread in the per-row kernel: cols <= 4 * 16 * 256

// ---------------------------------------------------------------------------------------
// per-row scale: one pass, row resident in registers
// ---------------------------------------------------------------------------------------
// kVmax: runs per thread (1, 2 or 4): the launcher spreads a row over as many threads as it has
// runs, so short rows cost few registers and more CTAs fit per SM.
template <typename T, int ROUND, int STORE4, int kVmax>
__global__ void __launch_bounds__(kThreads) row_ht_quant_rowscale_kernel(
    const T* __restrict__ x, int64_t rows, int cols, int64_t ldx, int n, QuantDev q, uint8_t* __restrict__ codes,
    int64_t ld_codes, float* __restrict__ scales, int tpr) {
  __shared__ float s_part[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rows_per_cta = kThreads / tpr;
  const int64_t row = (int64_t)blockIdx.x * rows_per_cta + threadIdx.x / tpr;
  const int t = threadIdx.x % tpr;
  const int nrun = cols >> 4;
  const int nv = (nrun + tpr - 1) / tpr;  // uniform over the CTA
  const bool row_ok = row < rows;
  const T* xr = x + (row_ok ? row : 0) * ldx;

  float2 v[kVmax][8];
  float mx = 0.0f;
#pragma unroll
  for (int j = 0; j < kVmax; ++j) {
    if (j < nv) {
      const int ri = t + j * tpr;
      if (row_ok && ri < nrun) Load16<T>::run(xr + (int64_t)ri * 16, v[j]);
      else zero16(v[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < kVmax; ++j) {
    if (j < nv) {
      butterfly16(v[j], n, lane);
      mx = fmaxf(mx, absmax16(v[j]));
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
      const int ri = t + j * tpr;
      if (ri < nrun) {
        const uint64_t e0 = (uint64_t)row * (uint64_t)cols + (uint64_t)ri * 16u;
        quantise_store16<ROUND, STORE4>(v[j], sp, q, e0, cr + (int64_t)ri * (STORE4 ? 8 : 16));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// per-tensor scale: pass 1 (abs-max) and pass 2 (quantise), streaming over 16-element runs
// ---------------------------------------------------------------------------------------
constexpr int kUnroll = 2;

// Where run `item` (row-major over rows x nrun) lives.  CONTIG: pitch == cols, so the tensor is
// one flat sequence of runs and no division is needed.
template <bool CONTIG>
__device__ __forceinline__ void locate(int64_t item, int nrun, int64_t ldx, int64_t ld_codes, int code_bytes,
                                       int64_t& x_off, int64_t& c_off) {
  if (CONTIG) {
    x_off = item * 16;
    c_off = item * code_bytes;
  } else {
    const int64_t row = item / nrun;
    const int ri = (int)(item - row * nrun);
    x_off = row * ldx + (int64_t)ri * 16;
    c_off = row * ld_codes + (int64_t)ri * code_bytes;
  }
}

template <typename T, bool CONTIG>
__global__ void __launch_bounds__(kThreads) row_ht_absmax_kernel(const T* __restrict__ x, int64_t rows, int cols,
                                                                 int64_t ldx, int n, uint32_t* __restrict__ absmax) {
  // blockIdx.y: sample of a batched call (rows = rows per sample, one abs-max word per sample)
  x += (int64_t)blockIdx.y * rows * ldx;
  absmax += blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int nrun = cols >> 4;
  const int64_t total = rows * nrun;
  const int64_t warp_id = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  float mx = 0.0f;
  for (int64_t base = warp_id * (32 * kUnroll); base < total; base += nwarps * (32 * kUnroll)) {
    float2 v[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t item = base + u * 32 + lane;
      if (item < total) {
        int64_t xo, co;
        locate<CONTIG>(item, nrun, ldx, 0, 0, xo, co);
        Load16<T>::run(x + xo, v[u]);
      } else {
        zero16(v[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      butterfly16(v[u], n, lane);
      mx = fmaxf(mx, absmax16(v[u]));
    }
  }
  mx = warp_max(mx);
  if (lane == 0) atomic_absmax(absmax, mx);
}

template <typename T, int ROUND, int STORE4, bool CONTIG>
__global__ void __launch_bounds__(kThreads) row_ht_quant_tensorscale_kernel(
    const T* __restrict__ x, int64_t rows, int cols, int64_t ldx, int n, QuantDev q, uint8_t* __restrict__ codes,
    int64_t ld_codes, float* __restrict__ scales, const uint32_t* __restrict__ absmax) {
  // blockIdx.y: sample of a batched call; the Philox / noise element index runs on across samples
  x += (int64_t)blockIdx.y * rows * ldx;
  codes += (int64_t)blockIdx.y * rows * ld_codes;
  scales += blockIdx.y;
  absmax += blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int nrun = cols >> 4;
  const int64_t total = rows * nrun;
  const uint64_t e_base = (uint64_t)blockIdx.y * (uint64_t)total * 16u;
  const int64_t warp_id = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const ScalePair sp = scale_from_absmax(__uint_as_float(*absmax), q.qmax);
  if (blockIdx.x == 0 && threadIdx.x == 0) scales[0] = sp.s;
  for (int64_t base = warp_id * (32 * kUnroll); base < total; base += nwarps * (32 * kUnroll)) {
    float2 v[kUnroll][8];
    int64_t coff[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t item = base + u * 32 + lane;
      coff[u] = -1;
      if (item < total) {
        int64_t xo;
        locate<CONTIG>(item, nrun, ldx, ld_codes, STORE4 ? 8 : 16, xo, coff[u]);
        Load16<T>::run(x + xo, v[u]);
      } else {
        zero16(v[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      butterfly16(v[u], n, lane);
      // logical element index of the run: row * cols + col == item * 16 in either layout
      if (coff[u] >= 0)
        quantise_store16<ROUND, STORE4>(v[u], sp, q, e_base + (uint64_t)(base + u * 32 + lane) * 16u, codes + coff[u]);
    }
  }
}

int grid_for(int64_t total_runs, int device_sms) {
  const int64_t per_cta = (int64_t)kThreads * kUnroll;
  int64_t want = (total_runs + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)device_sms * 8;  // 8 resident CTAs of 256 threads per SM
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}

template <typename T, int ROUND, int STORE4>
int launch_typed(const T* x, int64_t rows, int cols, int64_t ldx, int n, const hot_quant_t& hq, uint8_t* codes,
                 int64_t ld_codes, float* scales, uint32_t* absmax_ws, cudaStream_t st, int sms, int batch) {
  const QuantDev q = make_quant_dev(hq);
  if (hq.scale_mode == HOT_SCALE_ROW) {
    const int nrun = cols >> 4;
    int tpr = 32;
    while (tpr < kThreads && tpr < nrun) tpr <<= 1;  // one run per thread while a CTA can hold the row
    const int nv = (nrun + tpr - 1) / tpr;
    if (nv > kVmaxLimit)
      HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant: per-row scale supports cols <= %d (got %d)",
               kVmaxLimit * 16 * kThreads, cols);
    const int rows_per_cta = kThreads / tpr;
    const unsigned grid = (unsigned)((rows + rows_per_cta - 1) / rows_per_cta);
    if (nv == 1)
      row_ht_quant_rowscale_kernel<T, ROUND, STORE4, 1><<<grid, kThreads, 0, st>>>(x, rows, cols, ldx, n, q, codes, ld_codes, scales, tpr);
    else if (nv == 2)
      row_ht_quant_rowscale_kernel<T, ROUND, STORE4, 2><<<grid, kThreads, 0, st>>>(x, rows, cols, ldx, n, q, codes, ld_codes, scales, tpr);
    else
      row_ht_quant_rowscale_kernel<T, ROUND, STORE4, 4><<<grid, kThreads, 0, st>>>(x, rows, cols, ldx, n, q, codes, ld_codes, scales, tpr);
  } else {
    const dim3 grid((unsigned)grid_for(rows * (cols >> 4), (sms + batch - 1) / batch), (unsigned)batch);
    HOT_CUDA(cudaMemsetAsync(absmax_ws, 0, sizeof(uint32_t) * (size_t)batch, st));
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
                 int64_t ld_codes, float* scales, uint32_t* ws, cudaStream_t st, int sms, int batch) {
#define HOT_CASE(R, S)                                                                              \
  if (q.rounding == (R) && q.storage == (S))                                                        \
    return launch_typed<T, (R), (S)>(x, rows, cols, ldx, n, q, codes, ld_codes, scales, ws, st, sms, batch);
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

namespace hot {
namespace {
int row_ht_quant_impl(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order, const hot_quant_t* q,
                      void* codes, int64_t ld_codes, float* scales, uint32_t* absmax_ws, hot_stream_t stream, int batch) {
  if (rows == 0 && cols > 0 && q) return HOT_OK;  // nothing to do (and the pointers may be null)
  if (!x || !q || !codes || !scales) HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: null pointer");
  if (rows < 0 || cols <= 0) HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: bad shape %lld x %lld", (long long)rows, (long long)cols);
  if (int rc = validate_quant(q, "hot_row_ht_quant")) return rc;
  if (order < 1 || order > 64 || (order & (order - 1)))
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant: order %d not a power of two in [1, 64]", order);
  if (cols % 16 != 0 || cols % order != 0 || cols > (1 << 30))
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant: cols %lld must be a multiple of 16 and of the order %d",
             (long long)cols, order);
  const int esz = dtype == HOT_F32 ? 4 : 2;
  if (ldx < cols || (ldx * esz) % 16 != 0 || ((uintptr_t)x) % 16 != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: x and its pitch must be 16-byte aligned, ldx >= cols");
  const int64_t row_bytes = q->storage == HOT_STORE_INT4 ? cols / 2 : cols;
  if (ld_codes < row_bytes || ld_codes % 8 != 0 || (q->storage == HOT_STORE_INT8 && ld_codes % 16 != 0) ||
      ((uintptr_t)codes) % 16 != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: codes pitch %lld must be >= %lld and 16-byte aligned (8 for INT4)",
             (long long)ld_codes, (long long)row_bytes);
  if (q->scale_mode == HOT_SCALE_TENSOR && !absmax_ws) HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: absmax_ws is null");
  if (q->rounding == HOT_ROUND_STOCH_NOISE && ((uintptr_t)q->noise) % 16 != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant: noise must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int sms = device_sm_count();
  if (sms <= 0) return HOT_ERR_CUDA;
  if (dtype == HOT_F32)
    return launch_modes<float>((const float*)x, rows, (int)cols, ldx, order, *q, (uint8_t*)codes, ld_codes, scales,
                               absmax_ws, st, sms, batch);
  if (dtype == HOT_BF16)
    return launch_modes<__nv_bfloat16>((const __nv_bfloat16*)x, rows, (int)cols, ldx, order, *q, (uint8_t*)codes,
                                       ld_codes, scales, absmax_ws, st, sms, batch);
  HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant: dtype %d", dtype);
}
}  // namespace
}  // namespace hot

extern "C" int hot_row_ht_quant(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order,
                                const hot_quant_t* q, void* codes, int64_t ld_codes, float* scales,
                                uint32_t* absmax_ws, hot_stream_t stream) {
  return hot::row_ht_quant_impl(x, dtype, rows, cols, ldx, order, q, codes, ld_codes, scales, absmax_ws, stream, 1);
}

extern "C" int hot_row_ht_quant_batched(const void* x, int dtype, int64_t batch, int64_t rows, int64_t cols, int64_t ldx,
                                        int order, const hot_quant_t* q, void* codes, int64_t ld_codes, float* scales,
                                        uint32_t* absmax_ws, hot_stream_t stream) {
  using namespace hot;
  if (batch < 1 || batch > 65535) HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant_batched: batch %lld outside [1, 65535]", (long long)batch);
  if (!q) HOT_FAIL(HOT_ERR_ARG, "hot_row_ht_quant_batched: null pointer");
  if (q->scale_mode != HOT_SCALE_TENSOR)
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_row_ht_quant_batched: one scale per sample is HOT_SCALE_TENSOR; per-row scales do not depend on the batch");
  return row_ht_quant_impl(x, dtype, rows, cols, ldx, order, q, codes, ld_codes, scales, absmax_ws, stream, (int)batch);
}
