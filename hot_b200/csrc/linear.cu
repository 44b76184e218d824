// The HOT backward of one linear layer as a sequence of the three kernels, plus the
// forward-side activation-buffer compression.  All intermediates live in a caller-owned
// workspace; nothing here allocates or synchronises.
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace hot {

bool go_dual_supported(int64_t L, int64_t O, int64_t ldgo, int dtype, int order_o, int order_l, int rank_l,
                       const int32_t* sel_l, const hot_quant_t& q_gx, const hot_quant_t& q_gw);
int go_dual_quant(const void* go, int dtype, int64_t L, int64_t O, int64_t ldgo, int order_o, const int32_t* sel_l,
                  const hot_quant_t& q_gx, const hot_quant_t& q_gw, void* q_go, int64_t ld_qgo, float* s_gx, void* q_gw_t,
                  int64_t ld_qgw, float* s_gw, uint32_t* max_x, uint32_t* max_w, uint32_t* status, cudaStream_t st);

bool go_dual_tc_supported(int64_t L, int64_t O, int64_t ldgo, int dtype, int order_o, int order_l, int rank_l,
                          const int32_t* sel_l, const hot_quant_t& q_gx, const hot_quant_t& q_gw);
bool tc_weight_job_supported(int64_t O, int64_t I, int64_t ldw, const hot_quant_t& q_w);
int go_dual_quant_tc(const void* go, int64_t L, int64_t O, int64_t ldgo, const hot_quant_t& q_gx, const hot_quant_t& q_gw,
                     void* q_go, int64_t ld_qgo, float* s_gx, void* q_gw_t, int64_t ld_qgw, float* s_gw, uint32_t* max_x,
                     uint32_t* max_w, uint32_t* counters, size_t counter_words, uint32_t* status, cudaStream_t st,
                     const TcWeightJob* wj, bool col_only = false);
bool abc_tc_supported(int64_t L, int64_t I, int64_t ldx, int dtype, int order_l, int rank_l, const int32_t* sel_l,
                      const hot_quant_t& q_x);
int gemm_i8_dual_ws(const hot_gemm_problem_t* main_problem, const hot_gemm_problem_t* rider_problem, void* workspace,
                    size_t workspace_bytes, uint32_t* counters, uint32_t* status_word, hot_stream_t stream);

namespace {

// Which fused grad_out kernels serve a call: the tensor-core pair where it covers the configuration,
// else the butterfly pair.  HOT_GO_DUAL=butterfly keeps the tensor-core pair out (the parity tests
// compare the two).
bool use_tc(int64_t L, int64_t O, int64_t ldgo, const hot_linear_cfg_t& c) {
  const char* env = getenv("HOT_GO_DUAL");
  if (env && env[0] == 'b') return false;
  return go_dual_tc_supported(L, O, ldgo, c.dtype, c.order_o, c.order_l, c.rank_l, c.sel_l, c.q_gx, c.q_gw);
}

// counters: scratch words behind the abs-max words: two for the tensor-core pair's tile hand-out, and whatever else
// of the caller's lies behind them and is to be cleared along (counter_words in all; tensor-core pair only)
// wj: the weight that rides along; only with the tensor-core pair (see weight_rides)
int go_dual_any(const void* go, int64_t L, int64_t O, int64_t ldgo, const hot_linear_cfg_t& c, void* q_go, int64_t ld_qgo,
                float* s_gx, void* q_gw_t, int64_t ld_qgw, float* s_gw, uint32_t* max_x, uint32_t* max_w, uint32_t* counters,
                size_t counter_words, uint32_t* status, cudaStream_t st, const TcWeightJob* wj = nullptr) {
  if (use_tc(L, O, ldgo, c))
    return go_dual_quant_tc(go, L, O, ldgo, c.q_gx, c.q_gw, q_go, ld_qgo, s_gx, q_gw_t, ld_qgw, s_gw, max_x, max_w, counters,
                            counter_words, status, st, wj);
  if (wj) HOT_FAIL(HOT_ERR_ARG, "go_dual_quant: the weight rides along with the tensor-core kernels only");
  return go_dual_quant(go, c.dtype, L, O, ldgo, c.order_o, c.sel_l, c.q_gx, c.q_gw, q_go, ld_qgo, s_gx, q_gw_t, ld_qgw, s_gw,
                       max_x, max_w, status, st);
}

// A helper stream per device, so that the weight quantisation (independent of grad_out) runs
// beside the grad_out kernels.  Created on first use: make the first call on a device outside
// stream capture.  Fork and join are plain events, which also work under capture.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
SideStream g_side[kMaxDevices];
std::mutex g_side_mutex;  // guards creation only; the streams and events themselves are used by one caller at a time

int side_stream(SideStream** out) {
  int dev = -1;
  HOT_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_linear_backward: device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(g_side_mutex);
  SideStream& s = g_side[dev];
  if (!s.stream) {
    cudaStream_t st;
    cudaEvent_t f, j;
    HOT_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    HOT_CUDA(cudaEventCreateWithFlags(&f, cudaEventDisableTiming));
    HOT_CUDA(cudaEventCreateWithFlags(&j, cudaEventDisableTiming));
    s.fork = f;
    s.join = j;
    s.stream = st;
  }
  *out = &s;
  return HOT_OK;
}

constexpr size_t kAlign = 256;
constexpr int kRiderCounters = 160;  // one word per g_w tile that the dual GEMM may cut along K
inline size_t up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline int64_t code_pitch(int64_t len, int storage) { return (int64_t)up((size_t)(storage == HOT_STORE_INT4 ? (len + 1) / 2 : len), 16); }

struct Workspace {
  size_t off_qgo, off_sgo, off_qw, off_sw, off_qgw, off_sgw, off_scratch, w_scratch_off, off_gemm, gemm_bytes, total;
  int64_t ld_qgo, ld_qw, ld_qgw, lp;
};

int plan(int64_t L, int64_t O, int64_t I, const hot_linear_cfg_t& c, Workspace& w) {
  if (c.order_l < 1 || c.rank_l < 1 || c.rank_l > c.order_l || L % c.order_l != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_linear: tokens %lld not a multiple of the low-rank order %d (rank %d)", (long long)L,
             c.order_l, c.rank_l);
  w.lp = L / c.order_l * c.rank_l;
  w.ld_qgo = code_pitch(O, c.q_gx.storage);
  w.ld_qw = code_pitch(O, HOT_STORE_INT8);  // weight codes are kept one per byte (see hot_linear_backward)
  w.ld_qgw = code_pitch(w.lp, c.q_gw.storage);
  size_t o = 0;
  w.off_qgo = o; o += up((size_t)L * w.ld_qgo, kAlign);
  w.off_sgo = o; o += up((size_t)L * sizeof(float), kAlign);
  w.off_qw = o;  o += up((size_t)I * w.ld_qw, kAlign);
  w.off_sw = o;  o += kAlign;
  w.off_qgw = o; o += up((size_t)O * w.ld_qgw, kAlign);
  w.off_sgw = o; o += up((size_t)O * sizeof(float), kAlign);
  // scratch words: 64 fixed + per-token (L) + per-channel (O) maxima + 2 tile counters + kRiderCounters of the
  // GEMM + the weight quantiser's own
  w.w_scratch_off = (size_t)((64 + L + O + 2 + kRiderCounters + 1) / 2 * 2);
  w.off_scratch = o;
  o += up((w.w_scratch_off + hot_col_ht_quant_scratch_words(c.dtype, O, I, c.order_o, c.order_o, c.q_w.scale_mode) + 64) * sizeof(uint32_t), kAlign);
  // stream-K workspace of the two GEMMs (they run one after the other and share it)
  const size_t g1 = hot_gemm_i8_workspace_bytes(L, I), g2 = hot_gemm_i8_workspace_bytes(O, I);
  w.gemm_bytes = g1 > g2 ? g1 : g2;
  w.off_gemm = o; o += up(w.gemm_bytes, kAlign);
  w.total = o;
  return HOT_OK;
}

}  // namespace
}  // namespace hot

extern "C" size_t hot_linear_workspace_bytes(int64_t L, int64_t O, int64_t I, const hot_linear_cfg_t* cfg) {
  hot::Workspace w;
  if (!cfg || L <= 0 || O <= 0 || I <= 0 || hot::plan(L, O, I, *cfg, w)) return 0;
  return w.total;
}

extern "C" int64_t hot_abc_pitch(int64_t L, const hot_linear_cfg_t* cfg) {
  if (!cfg || cfg->order_l < 1 || L % cfg->order_l != 0) return 0;
  return hot::code_pitch(L / cfg->order_l * cfg->rank_l, cfg->q_x.storage);
}

extern "C" int hot_abc_compress(const void* x, int64_t L, int64_t I, int64_t ldx, const hot_linear_cfg_t* cfg,
                                void* x_q_t, float* scale_x, void* workspace, size_t workspace_bytes,
                                hot_stream_t stream) {
  using namespace hot;
  if (!x || !cfg || !x_q_t || !scale_x || !workspace) HOT_FAIL(HOT_ERR_ARG, "hot_abc_compress: null pointer");
  if (cfg->q_x.scale_mode == HOT_SCALE_ROW) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_abc_compress: the activation buffer takes one scale");
  const size_t need = 4 * hot_col_ht_quant_scratch_words(cfg->dtype, L, I, cfg->order_l, cfg->rank_l, cfg->q_x.scale_mode);
  if (need == 0 || workspace_bytes < need || ((uintptr_t)workspace) % 8 != 0)
    HOT_FAIL(HOT_ERR_WORKSPACE, "hot_abc_compress: workspace needs %zu bytes, 8-byte aligned (got %zu)", need, workspace_bytes);
  const int64_t pitch = hot_abc_pitch(L, cfg);
  if (pitch == 0) HOT_FAIL(HOT_ERR_ARG, "hot_abc_compress: tokens %lld not a multiple of the low-rank order %d", (long long)L, cfg->order_l);
  // bf16 with the order-16 token basis: the token side of the tensor-core grad_out kernels on its own (same codes as
  // the butterfly kernel below unless a 16-term sum is inexact in fp32; HOT_ABC=butterfly keeps that kernel).
  // Workspace words: 0 abs-max, 1-2 tile counters, 3 status (non-zero afterwards: a device-side wait ran out).
  const char* abc_env = getenv("HOT_ABC");
  if (workspace_bytes >= 16 && !(abc_env && abc_env[0] == 'b') && pitch % 16 == 0 && ((uintptr_t)x_q_t) % 16 == 0 &&
      ((uintptr_t)x) % 16 == 0 && abc_tc_supported(L, I, ldx, cfg->dtype, cfg->order_l, cfg->rank_l, cfg->sel_l, cfg->q_x)) {
    if (int rc = validate_quant(&cfg->q_x, "hot_abc_compress")) return rc;
    uint32_t* wsw = (uint32_t*)workspace;
    return go_dual_quant_tc(x, L, I, ldx, cfg->q_x, cfg->q_x, nullptr, 0, nullptr, x_q_t, pitch, scale_x, nullptr, wsw, wsw + 1, 3, wsw + 3,
                            (cudaStream_t)stream, nullptr, true);
  }
  return hot_col_ht_quant(x, cfg->dtype, L, I, ldx, cfg->order_l, cfg->sel_l, cfg->rank_l, &cfg->q_x, HOT_LAYOUT_NATURAL,
                          x_q_t, pitch, scale_x, (uint32_t*)workspace, stream);
}

extern "C" int hot_go_dual_quant(const void* go, int64_t L, int64_t O, int64_t ldgo, const hot_linear_cfg_t* cfg, void* q_go,
                                 int64_t ld_qgo, float* s_gx, void* q_gw_t, int64_t ld_qgw, float* s_gw,
                                 uint32_t* scratch, uint32_t* status_word, hot_stream_t stream) {
  using namespace hot;
  if (!go || !cfg || !q_go || !s_gx || !q_gw_t || !s_gw || !scratch) HOT_FAIL(HOT_ERR_ARG, "hot_go_dual_quant: null pointer");
  if (L <= 0 || O <= 0) HOT_FAIL(HOT_ERR_ARG, "hot_go_dual_quant: bad shape");
  if (int rc = validate_quant(&cfg->q_gx, "hot_go_dual_quant")) return rc;
  if (int rc = validate_quant(&cfg->q_gw, "hot_go_dual_quant")) return rc;
  if (!go_dual_supported(L, O, ldgo, cfg->dtype, cfg->order_o, cfg->order_l, cfg->rank_l, cfg->sel_l, cfg->q_gx, cfg->q_gw))
    HOT_FAIL(HOT_ERR_UNSUPPORTED,
             "hot_go_dual_quant covers: low-rank basis = 8 lowest-sequency rows of H_16, tokens %% 32 == 0, channels %% 64 == 0, "
             "INT8 storage on the g_w side, nearest or Philox rounding");
  const int64_t need_x = cfg->q_gx.storage == HOT_STORE_INT4 ? O / 2 : O;
  if (ld_qgo < need_x || ld_qgo % 16 || ld_qgw < L / 2 || ld_qgw % 16 || ((uintptr_t)q_go) % 16 || ((uintptr_t)q_gw_t) % 16 ||
      ((uintptr_t)go) % 16)
    HOT_FAIL(HOT_ERR_ARG, "hot_go_dual_quant: buffers and pitches must be 16-byte aligned and cover the codes");
  return go_dual_any(go, L, O, ldgo, *cfg, q_go, ld_qgo, s_gx, q_gw_t, ld_qgw, s_gw, scratch, scratch + L, scratch + L + O, 2, status_word,
                     (cudaStream_t)stream);
}

extern "C" int hot_linear_backward(const void* go, int64_t ldgo, const void* w, int64_t ldw, const void* x_q_t,
                                   const float* scale_x, int64_t L, int64_t O, int64_t I, const hot_linear_cfg_t* cfg,
                                   void* grad_x, int64_t ldgx, void* grad_w, int64_t ldgw, void* workspace,
                                   size_t workspace_bytes, uint32_t* status_word, hot_stream_t stream) {
  using namespace hot;
  if (!go || !w || !x_q_t || !scale_x || !cfg || !workspace) HOT_FAIL(HOT_ERR_ARG, "hot_linear_backward: null pointer");
  if (!grad_x && !grad_w) HOT_FAIL(HOT_ERR_ARG, "hot_linear_backward: no output requested");
  if (L <= 0 || O <= 0 || I <= 0) HOT_FAIL(HOT_ERR_ARG, "hot_linear_backward: bad shape");
  Workspace ws;
  if (int rc = plan(L, O, I, *cfg, ws)) return rc;
  if (workspace_bytes < ws.total)
    HOT_FAIL(HOT_ERR_WORKSPACE, "hot_linear_backward: workspace %zu < %zu bytes", workspace_bytes, ws.total);
  if (((uintptr_t)workspace) % kAlign != 0) HOT_FAIL(HOT_ERR_ARG, "hot_linear_backward: workspace must be 256-byte aligned");
  if (cfg->order_o < 1 || cfg->order_o > 16 || O % cfg->order_o != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_linear_backward: order_o %d does not divide O = %lld", cfg->order_o, (long long)O);
  // the scratch plan reserves abs-max words for the two grad_out quantisers; the two-moment clip needs
  // words per CTA instead and is what the reference offers for the weight and the activation only
  if (cfg->q_gx.scale_mode == HOT_SCALE_SAWB || cfg->q_gw.scale_mode == HOT_SCALE_SAWB)
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_linear_backward: HOT_SCALE_SAWB is for the weight and the activation buffer, not for grad_out");
  uint8_t* base = (uint8_t*)workspace;
  // scratch words: [0, 64) per-tensor maxima of the three quantiser calls and the weight's,
  // then per-token (L) and per-channel (O) maxima
  uint32_t* scratch = (uint32_t*)(base + ws.off_scratch);
  float* s_go = (float*)(base + ws.off_sgo);
  float* s_w = (float*)(base + ws.off_sw);
  float* s_gw = (float*)(base + ws.off_sgw);
  int rc;
  // grad_out: one fused pair of kernels serves both operands when both gradients are wanted and
  // the configuration is the one they cover; otherwise each side runs its own kernel
  const bool dual = grad_x && grad_w &&
                    go_dual_supported(L, O, ldgo, cfg->dtype, cfg->order_o, cfg->order_l, cfg->rank_l, cfg->sel_l, cfg->q_gx,
                                      cfg->q_gw);
  // The weight: where the tensor-core grad_out kernels run, they transform and quantise it on the side (no launch
  // of its own); else it starts first, on the helper stream.  HOT_WEIGHT_QUANT=separate keeps it apart (the parity
  // tests compare the two).
  SideStream* side = nullptr;
  cudaStream_t main_st = (cudaStream_t)stream;
  hot_quant_t q_w8 = cfg->q_w;
  q_w8.storage = HOT_STORE_INT8;
  const char* wq_env = getenv("HOT_WEIGHT_QUANT");
  const bool weight_rides = grad_x && dual && use_tc(L, O, ldgo, *cfg) && cfg->q_w.scale_mode == HOT_SCALE_TENSOR &&
                            tc_weight_job_supported(O, I, ldw, q_w8) && !(wq_env && wq_env[0] == 's');
  const TcWeightJob wj = {w, ldw, I, q_w8, base + ws.off_qw, ws.ld_qw, s_w, scratch + ws.w_scratch_off};
  if (grad_x && !weight_rides) {
    if (cfg->q_w.scale_mode == HOT_SCALE_ROW) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_linear_backward: the weight takes one scale");
    if ((rc = side_stream(&side))) return rc;
    HOT_CUDA(cudaEventRecord(side->fork, main_st));
    HOT_CUDA(cudaStreamWaitEvent(side->stream, side->fork, 0));
    int32_t ident[64];
    for (int i = 0; i < 64; ++i) ident[i] = i;
    // The quantised weight is the B operand of every CTA of the g_x GEMM and is tiny (O * I bytes):
    // it is stored one code per byte whatever its bit width, so that it reaches the tensor core by
    // TMA alone and only grad_out (the large, streamed operand) is expanded in shared memory.
    rc = hot_col_ht_quant(w, cfg->dtype, O, I, ldw, cfg->order_o, ident, cfg->order_o, &q_w8, HOT_LAYOUT_NATURAL,
                          base + ws.off_qw, ws.ld_qw, s_w, scratch + ws.w_scratch_off, (hot_stream_t)side->stream);
    cudaEventRecord(side->join, side->stream);
    if (rc) {
      cudaStreamWaitEvent(main_st, side->join, 0);  // rejoin, so that a capture in progress stays well-formed
      return rc;
    }
  }
  bool joined = side == nullptr;
  auto rejoin = [&]() {
    if (!joined) cudaStreamWaitEvent(main_st, side->join, 0);
    joined = true;
  };
  if (dual) {
    rc = go_dual_any(go, L, O, ldgo, *cfg, base + ws.off_qgo, ws.ld_qgo, s_go, base + ws.off_qgw, ws.ld_qgw, s_gw, scratch + 64,
                     scratch + 64 + L, scratch + 64 + L + O, 2 + kRiderCounters, status_word, (cudaStream_t)stream,
                     weight_rides ? &wj : nullptr);
    if (rc) {
      rejoin();
      return rc;
    }
  }
  if (grad_x && !dual) {
    rc = hot_row_ht_quant(go, cfg->dtype, L, O, ldgo, cfg->order_o, &cfg->q_gx, base + ws.off_qgo, ws.ld_qgo, s_go, scratch,
                          stream);
    if (rc) {
      rejoin();
      return rc;
    }
  }
  if (grad_w && !dual) {
    rc = hot_col_ht_quant(go, cfg->dtype, L, O, ldgo, cfg->order_l, cfg->sel_l, cfg->rank_l, &cfg->q_gw,
                          HOT_LAYOUT_TRANSPOSED, base + ws.off_qgw, ws.ld_qgw, s_gw, scratch + 64 + L, stream);
    if (rc) {
      rejoin();
      return rc;
    }
  }
  rejoin();  // the g_x GEMM needs the quantised weight
  const float post_x = 1.0f / (float)cfg->order_o, post_w = 1.0f / (float)cfg->order_l;
  const int gx_row = cfg->q_gx.scale_mode == HOT_SCALE_ROW, gw_row = cfg->q_gw.scale_mode == HOT_SCALE_ROW;
  if (grad_x && grad_w && cfg->q_gw.storage == HOT_STORE_INT8 && cfg->q_x.storage == HOT_STORE_INT8) {
    // both products in one launch: the few long g_w tiles run in the SMs that the last wave of g_x tiles leaves idle
    hot_gemm_problem_t gx = {base + ws.off_qgo, cfg->q_gx.storage, ws.ld_qgo, base + ws.off_qw, ws.ld_qw, L, I, O, s_go, gx_row,
                             s_w, 0, post_x, grad_x, cfg->dtype, ldgx};
    hot_gemm_problem_t gw = {base + ws.off_qgw, HOT_STORE_INT8, ws.ld_qgw, x_q_t, hot_abc_pitch(L, cfg), O, I, ws.lp, s_gw, gw_row,
                             scale_x, 0, post_w, grad_w, cfg->dtype, ldgw};
    // the GEMM's counters lie behind the tile counters of the tensor-core grad_out kernels, which clear them along
    uint32_t* rider_counters = scratch + 64 + L + O + 2;
    if (!(dual && use_tc(L, O, ldgo, *cfg))) HOT_CUDA(cudaMemsetAsync(rider_counters, 0, kRiderCounters * sizeof(uint32_t), main_st));
    return gemm_i8_dual_ws(&gx, &gw, ws.gemm_bytes ? base + ws.off_gemm : nullptr, ws.gemm_bytes, rider_counters, status_word, stream);
  }
  if (grad_x) {
    rc = hot_gemm_i8_ws(base + ws.off_qgo, cfg->q_gx.storage, ws.ld_qgo, base + ws.off_qw, HOT_STORE_INT8, ws.ld_qw, L, I, O,
                        s_go, gx_row, s_w, 0, post_x, grad_x, cfg->dtype, ldgx, ws.gemm_bytes ? base + ws.off_gemm : nullptr,
                        ws.gemm_bytes, status_word, stream);
    if (rc) return rc;
  }
  if (grad_w) {
    rc = hot_gemm_i8_ws(base + ws.off_qgw, cfg->q_gw.storage, ws.ld_qgw, x_q_t, cfg->q_x.storage, hot_abc_pitch(L, cfg), O, I,
                        ws.lp, s_gw, gw_row, scale_x, 0, post_w, grad_w, cfg->dtype, ldgw,
                        ws.gemm_bytes ? base + ws.off_gemm : nullptr, ws.gemm_bytes, status_word, stream);
    if (rc) return rc;
  }
  return HOT_OK;
}
