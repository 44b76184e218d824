// Host-side plumbing shared by the entry points: last-error text, argument validation,
// device properties.
#include <cstdarg>
#include <cstdio>

#include "tma.cuh"

namespace hot {

namespace {
thread_local char g_last_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int validate_quant(const hot_quant_t* q, const char* who) {
  if (q->bits < 2 || q->bits > 8) HOT_FAIL(HOT_ERR_ARG, "%s: bits %d outside [2, 8]", who, q->bits);
  if (q->storage != HOT_STORE_INT8 && q->storage != HOT_STORE_INT4) HOT_FAIL(HOT_ERR_ARG, "%s: storage %d", who, q->storage);
  if (q->storage == HOT_STORE_INT4 && q->bits > 4) HOT_FAIL(HOT_ERR_ARG, "%s: INT4 storage needs bits <= 4 (got %d)", who, q->bits);
  if (q->rounding < HOT_ROUND_NEAREST || q->rounding > HOT_ROUND_STOCH_NOISE) HOT_FAIL(HOT_ERR_ARG, "%s: rounding %d", who, q->rounding);
  if (q->scale_mode != HOT_SCALE_TENSOR && q->scale_mode != HOT_SCALE_ROW && q->scale_mode != HOT_SCALE_SAWB) HOT_FAIL(HOT_ERR_ARG, "%s: scale_mode %d", who, q->scale_mode);
  if (q->rounding == HOT_ROUND_STOCH_NOISE && !q->noise) HOT_FAIL(HOT_ERR_ARG, "%s: explicit-noise rounding without a noise pointer", who);
  return HOT_OK;
}

namespace {
std::atomic<uint64_t> g_wait_limit_ns{1500ull * 1000ull * 1000ull};
}
uint64_t wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }
void set_wait_limit_ns(uint64_t ns) { g_wait_limit_ns.store(ns, std::memory_order_relaxed); }

namespace {
std::atomic<int> g_sm_margin{0};
}
void set_sm_margin(int sms) { g_sm_margin.store(sms < 0 ? 0 : sms, std::memory_order_relaxed); }

// SMs the persistent kernels size their grids to: those of the current device, less the margin a caller
// asked to be left free (for a communication library's kernels that run beside them).
int device_sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    set_error("cannot query the current CUDA device");
    return -1;
  }
  const int left = sms - g_sm_margin.load(std::memory_order_relaxed);
  return left < 1 ? 1 : left;
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn resolve_encode_fn() {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    return reinterpret_cast<EncodeTiledFn>(ptr);
  return nullptr;
}

EncodeTiledFn encode_fn() {
  static const EncodeTiledFn fn = resolve_encode_fn();  // initialised once, thread-safe
  return fn;
}

// Tensor map over a [rows, row_bytes] byte matrix with pitch ld, box = box_bytes x box_rows.
}  // namespace

int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int64_t ld, int box_bytes,
             int box_rows, int swizzle_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) HOT_FAIL(HOT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) HOT_FAIL(HOT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return HOT_OK;
}


}  // namespace hot

extern "C" const char* hot_status_string(int status) {
  switch (status) {
    case HOT_OK: return "ok";
    case HOT_ERR_ARG: return "invalid argument";
    case HOT_ERR_UNSUPPORTED: return "unsupported size or mode";
    case HOT_ERR_CUDA: return "CUDA call failed";
    case HOT_ERR_TIMEOUT: return "bounded device-side wait ran out";
    case HOT_ERR_WORKSPACE: return "workspace too small";
  }
  return "unknown status";
}

extern "C" const char* hot_last_error(void) { return hot::g_last_error; }

extern "C" int hot_abi_version(void) { return 1; }
