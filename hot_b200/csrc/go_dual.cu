// grad_output feeds both halves of the backward: Hadamard along the channels + INT4 for g_x,
// Hadamard low-rank along the tokens + INT8 for g_w.  These kernels serve both from ONE read of
// each tile: a persistent CTA streams 256-token x 64-channel tiles through a two-stage
// shared-memory ring filled by TMA (the next tile is in flight while this one is processed);
// a row phase takes 16-channel runs of a token, a column phase takes two 16-token blocks of a
// channel pair, both with packed fp32 butterflies in registers.
//
//   pass 1  (dual_stats)  abs-max of both transformed tensors (per tensor, per token, per channel)
//   pass 2  (dual_quant)  the same transforms again, quantised against those abs-maxima:
//                         q_go [L, O] (INT4 packed or INT8) and q_gw^T [O, L/2] (INT8, written
//                         through a shared-memory transpose so rows go out in 128-byte pieces)
//
// Arithmetic, rounding and Philox indexing are those of row_ht_quant / col_ht_quant, so the
// outputs are bit-identical to running those two kernels one after the other.  Covered here:
// the token-side basis "8 lowest-sequency rows of H_16", channels a multiple of 64, tokens a multiple of 32,
// nearest or Philox rounding; everything else takes the separate kernels.
#include "ht_device.cuh"
#include "tma.cuh"

namespace hot {
namespace {

constexpr int kThreads = 256;
constexpr int kTT = 256;  // tokens per tile
constexpr int kTC = 64;   // channels per tile
constexpr int kStagePitch = 144;  // bytes per channel row of the transposed INT8 staging (128 used)

struct DualParams {
  int64_t L;
  int O;
  int n_o;                 // Hadamard order along channels (1..64)
  int x_row, w_row;        // per-token scale on the g_x side, per-channel scale on the g_w side
  int x_store4;            // g_x codes packed INT4
  QuantDev qx, qw;
  uint8_t* q_go;
  int64_t ld_qgo;
  uint8_t* q_gw;
  int64_t ld_qgw;
  float* s_x;              // [1] or [L]
  float* s_w;              // [1] or [O]
  uint32_t* max_x;         // [1] or [L]
  uint32_t* max_w;         // [1] or [O]
  uint32_t* status;
  uint64_t wait_ns;        // time limit of a device-side wait
};

template <typename T>
struct Tile {
  static constexpr int kRowBytes = kTC * (int)sizeof(T);
  static constexpr int kBytes = kTT * kRowBytes;
};

// 16 consecutive channels of one token from the shared-memory tile -> eight (A_i, B_i) pairs
template <typename T>
__device__ __forceinline__ void lds_run16(const uint8_t* p, float2 (&v)[8]);
template <>
__device__ __forceinline__ void lds_run16<float>(const uint8_t* p, float2 (&v)[8]) {
  const float4* q = reinterpret_cast<const float4*>(p);
  const float4 a0 = q[0], a1 = q[1], b0 = q[2], b1 = q[3];
  v[0] = make_float2(a0.x, b0.x); v[1] = make_float2(a0.y, b0.y);
  v[2] = make_float2(a0.z, b0.z); v[3] = make_float2(a0.w, b0.w);
  v[4] = make_float2(a1.x, b1.x); v[5] = make_float2(a1.y, b1.y);
  v[6] = make_float2(a1.z, b1.z); v[7] = make_float2(a1.w, b1.w);
}
template <>
__device__ __forceinline__ void lds_run16<__nv_bfloat16>(const uint8_t* p, float2 (&v)[8]) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
  const uint4 a = q[0], b = q[1];
  const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[2 * k] = make_float2(__uint_as_float(wa[k] << 16), __uint_as_float(wb[k] << 16));
    v[2 * k + 1] = make_float2(__uint_as_float(wa[k] & 0xFFFF0000u), __uint_as_float(wb[k] & 0xFFFF0000u));
  }
}

// Two adjacent channels (c, c + 1) of one token -> (x_c, x_c+1)
template <typename T>
__device__ __forceinline__ float2 lds_pair(const uint8_t* p);
template <>
__device__ __forceinline__ float2 lds_pair<float>(const uint8_t* p) {
  return *reinterpret_cast<const float2*>(p);
}
template <>
__device__ __forceinline__ float2 lds_pair<__nv_bfloat16>(const uint8_t* p) {
  const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}

// The token-side basis these kernels serve: the 8 lowest-sequency rows of H_16.  In natural
// (Sylvester) order those are the even rows 0, 2, ..., 14; output slot of natural row 2i:
__device__ constexpr int kSlotOfEvenRow[8] = {0, 7, 3, 4, 1, 6, 2, 5};
constexpr int kHalf16Sel[8] = {0, 8, 12, 4, 6, 14, 10, 2};  // natural row of output slot j

// Quantise 16 consecutive codes of two neighbouring rows (channels c, c + 1) of the transposed g_w
// operand into 16 bytes each.  y[i] = (value i of channel c, value i of channel c + 1): the packed
// fp32 operations run across the channel pair, so the transform's outputs are used where they are.
// e_a / e_b: stored-layout element index of the first code of each row (multiples of 16).
template <int ROUND>
__device__ __forceinline__ void quantise16_int8_pair(const float2 (&y)[16], const ScalePair& sa, const ScalePair& sb,
                                                     const QuantDev& q, uint64_t e_a, uint64_t e_b, uint4& out_a, uint4& out_b) {
  uint32_t wa[4] = {0, 0, 0, 0}, wb[4] = {0, 0, 0, 0};
  if (ROUND == HOT_ROUND_STOCH_PHILOX) {
    const bool rb4 = rand_bits(q.qmax) == 4;
    const float2 mk2 = make_float2(sa.mk, sb.mk), ck2 = make_float2(sa.ck, sb.ck);  // one divisor per channel
    uint32_t ka[2][8], kb[2][8];  // [first / second eight codes][i]: K bits of channel c / c + 1
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 t = __ffma2_rn(y[i], mk2, ck2);
      ka[i >> 3][i & 7] = __float_as_uint(t.x);
      kb[i >> 3][i & 7] = __float_as_uint(t.y);
    }
    philox_run16(ka[0], ka[1], q, e_a, rb4, wa[0], wa[1], wa[2], wa[3]);
    philox_run16(kb[0], kb[1], q, e_b, rb4, wb[0], wb[1], wb[2], wb[3]);
    const uint32_t off = (uint32_t)(q.qmax + 1.0f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (rb4) {
        wa[k] = (wa[k] >> 4) & 0x0F0F0F0Fu;
        wb[k] = (wb[k] >> 4) & 0x0F0F0F0Fu;
      }
      wa[k] = remove_offset(wa[k], off, 0x01010101u, 0x100u);
      wb[k] = remove_offset(wb[k], off, 0x01010101u, 0x100u);
    }
  } else {
    const int qmax = (int)q.qmax;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      wa[i >> 2] |= (uint32_t)(quantise_one<ROUND>(y[i].x, sa, 0.0f, qmax) & 0xFF) << (8 * (i & 3));
      wb[i >> 2] |= (uint32_t)(quantise_one<ROUND>(y[i].y, sb, 0.0f, qmax) & 0xFF) << (8 * (i & 3));
    }
  }
  out_a = make_uint4(wa[0], wa[1], wa[2], wa[3]);
  out_b = make_uint4(wb[0], wb[1], wb[2], wb[3]);
}

// PASS 0: statistics.  PASS 1: quantise (RX / RW: rounding of the g_x / g_w side).
// FAST: the configuration of the training path (channel order 16, one scale per tensor on both
// sides; X4: g_x codes packed INT4 or one per byte) with those choices folded at compile time;
// otherwise they are read from the parameters.
template <typename T, int PASS, int RX, int RW, bool FAST, bool X4>
__global__ void __launch_bounds__(kThreads, sizeof(T) == 2 ? 3 : 1) go_dual_kernel(const __grid_constant__ CUtensorMap tmap, DualParams p) {
  const int n_o = FAST ? 16 : p.n_o;
  const bool x_row = FAST ? false : p.x_row != 0;
  const bool w_row = FAST ? false : p.w_row != 0;
  const bool x_store4 = FAST ? X4 : p.x_store4 != 0;
  extern __shared__ uint8_t smem_raw[];
  // rounded up to 128 bytes by an offset, so that every pointer below is still visibly derived from
  // the shared array and its loads and stores compile to shared-memory instructions
  uint8_t* smem = smem_raw + ((128u - ((uint32_t)__cvta_generic_to_shared(smem_raw) & 127u)) & 127u);
  uint8_t* stage_out = smem + 2 * Tile<T>::kBytes;                       // [kTC][kStagePitch] (PASS 1)
  uint32_t* s_colmax = reinterpret_cast<uint32_t*>(stage_out);          // [kTC]             (PASS 0)
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + 2 * Tile<T>::kBytes + kTC * kStagePitch);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(full + 2);

  const int tid = threadIdx.x, lane = tid & 31;
  const int tiles_c = p.O / kTC;
  const int tiles_t = (int)((p.L + kTT - 1) / kTT);
  const int num_tiles = tiles_c * tiles_t;

  if (tid == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tma_prefetch_desc(&tmap);
  }
  __syncthreads();
  // tile index -> (token tile, channel tile): channel tiles fastest, so that neighbouring CTAs
  // work on the same token rows
  auto issue = [&](int tile_idx, int s) {
    const int tt = tile_idx / tiles_c, tc = tile_idx % tiles_c;
    mbar_expect_tx(&full[s], Tile<T>::kBytes);
    tma_load_2d(smem + s * Tile<T>::kBytes, &tmap, &full[s], tc * Tile<T>::kRowBytes, tt * kTT);
  };
  if (tid == 0 && (int)blockIdx.x < num_tiles) issue(blockIdx.x, 0);

  ScalePair sp_x = scale_from_absmax(0.0f, p.qx.qmax), sp_w = scale_from_absmax(0.0f, p.qw.qmax);
  if (PASS == 1) {
    // launched as a programmatic dependent of the statistics pass: everything above (barriers, the
    // first tile's load of grad_out, which that pass does not write) ran while it drained; its
    // abs-maxima are visible once this returns
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!x_row) sp_x = scale_from_absmax(__uint_as_float(p.max_x[0]), p.qx.qmax);
    if (!w_row) sp_w = scale_from_absmax(__uint_as_float(p.max_w[0]), p.qw.qmax);
    if (blockIdx.x == 0 && tid == 0) {
      if (!x_row) p.s_x[0] = sp_x.s;
      if (!w_row) p.s_w[0] = sp_w.s;
    }
  }
  float tmax_x = 0.0f, tmax_w = 0.0f;  // per-tensor maxima of this thread (PASS 0)

  uint32_t it = 0;
  bool ok = true;
  for (int t_idx = blockIdx.x; t_idx < num_tiles; t_idx += gridDim.x, ++it) {
    const int s = it & 1;
    const int next = t_idx + gridDim.x;
    if (tid == 0 && next < num_tiles) issue(next, s ^ 1);  // stage s^1 was released by the barrier below
    // the whole CTA leaves the tile loop together when a wait ran out (a thread that saw the barrier complete
    // in time must not go on to the __syncthreads below while others have left)
    ok = __syncthreads_and(mbar_wait(&full[s], (it >> 1) & 1u, abort_flag, p.wait_ns)) != 0;
    if (!ok) break;
    const uint8_t* tl = smem + s * Tile<T>::kBytes;
    const int tt = t_idx / tiles_c, tc = t_idx % tiles_c;
    const int64_t tok0 = (int64_t)tt * kTT;
    const int ch0 = tc * kTC;

    if (PASS == 0 && w_row) {
      if (tid < kTC) s_colmax[tid] = 0u;
      __syncthreads();
    }

    // ---- row phase: 16-channel runs; run r of token k is item 4k + r (adjacent lanes) -------
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float2 v[2][8];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int item = tid + (half * 2 + u) * kThreads;
        lds_run16<T>(tl + (item >> 2) * Tile<T>::kRowBytes + (item & 3) * 16 * (int)sizeof(T), v[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int item = tid + (half * 2 + u) * kThreads;
        const int64_t tok = tok0 + (item >> 2);
        const int ch = ch0 + (item & 3) * 16;
        butterfly16(v[u], n_o, lane);
        if (PASS == 0) {
          float m = absmax16(v[u]);
          if (x_row) {
            m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
            if ((lane & 3) == 0 && tok < p.L) atomic_absmax(p.max_x + tok, m);
          } else {
            tmax_x = fmaxf(tmax_x, m);
          }
        } else if (tok < p.L) {
          ScalePair sp = sp_x;
          if (x_row) {
            sp = scale_from_absmax(__uint_as_float(p.max_x[tok]), p.qx.qmax);
            if (tc == 0 && (item & 3) == 0) p.s_x[tok] = sp.s;
          }
          const uint64_t e0 = (uint64_t)tok * (uint64_t)p.O + (uint64_t)ch;
          uint8_t* dst = p.q_go + tok * p.ld_qgo + (x_store4 ? (ch >> 1) : ch);
          if (x_store4) quantise_store16<RX, 1>(v[u], sp, p.qx, e0, dst);
          else quantise_store16<RX, 0>(v[u], sp, p.qx, e0, dst);
        }
      }
    }

    // ---- column phase: channel pair cp (lane), token blocks 2*bp and 2*bp+1 (warp) ----------
    {
      const int cp = tid & 31, bp = tid >> 5;
      const int c_loc = cp * 2;
      float2 y[16];  // kept rows of the channel pair: block A slots 0..7 | block B slots 0..7
      float cmax0 = 0.0f, cmax1 = 0.0f;
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        float2 u[16], e[8];
        const uint8_t* base = tl + (bp * 32 + blk * 16) * Tile<T>::kRowBytes + c_loc * (int)sizeof(T);
#pragma unroll
        for (int t = 0; t < 16; ++t) u[t] = lds_pair<T>(base + t * Tile<T>::kRowBytes);
        butterfly_tokens16_even(u, e);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (PASS == 0) {
            cmax0 = fmaxf(cmax0, fabsf(e[i].x));
            cmax1 = fmaxf(cmax1, fabsf(e[i].y));
          } else {
            y[blk * 8 + kSlotOfEvenRow[i]] = e[i];
          }
        }
      }
      const int64_t blk_pair = tok0 / 32 + bp;           // global index of this pair of token blocks
      const bool pair_ok = tok0 + bp * 32 < p.L;          // tokens are a multiple of 32: all or nothing
      if (PASS == 0) {
        if (w_row) {
          atomicMax(&s_colmax[c_loc], __float_as_uint(cmax0));
          atomicMax(&s_colmax[c_loc + 1], __float_as_uint(cmax1));
        } else {
          tmax_w = fmaxf(tmax_w, fmaxf(cmax0, cmax1));
        }
      } else {
        const int64_t out_len = p.L / 2;
        const int ch = ch0 + c_loc;
        ScalePair sa = sp_w, sb = sp_w;
        if (w_row) {
          sa = scale_from_absmax(__uint_as_float(p.max_w[ch]), p.qw.qmax);
          sb = scale_from_absmax(__uint_as_float(p.max_w[ch + 1]), p.qw.qmax);
          if (tt == 0 && bp == 0) {
            p.s_w[ch] = sa.s;
            p.s_w[ch + 1] = sb.s;
          }
        }
        uint4 codes_a = make_uint4(0, 0, 0, 0), codes_b = make_uint4(0, 0, 0, 0);
        if (pair_ok) {
          const uint64_t e_a = (uint64_t)ch * (uint64_t)out_len + (uint64_t)blk_pair * 16u;
          quantise16_int8_pair<RW>(y, sa, sb, p.qw, e_a, e_a + (uint64_t)out_len, codes_a, codes_b);
        }
        *reinterpret_cast<uint4*>(stage_out + c_loc * kStagePitch + bp * 16) = codes_a;
        *reinterpret_cast<uint4*>(stage_out + (c_loc + 1) * kStagePitch + bp * 16) = codes_b;
      }
    }
    __syncthreads();  // tile consumed; staging complete
    if (PASS == 0) {
      if (w_row && tid < kTC) atomicMax(p.max_w + ch0 + tid, s_colmax[tid]);
    } else {
      // transposed g_w codes of this tile: kTC rows x 128 bytes, written in 16-byte pieces
      const int64_t pos0 = tok0 / 2;                       // first stored position of the tile in a row
      const int64_t out_len = p.L / 2;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int idx = tid + k * kThreads;
        const int c = idx >> 3, piece = idx & 7;
        if (pos0 + piece * 16 < out_len)
          *reinterpret_cast<uint4*>(p.q_gw + (int64_t)(ch0 + c) * p.ld_qgw + pos0 + piece * 16) =
              *reinterpret_cast<const uint4*>(stage_out + c * kStagePitch + piece * 16);
      }
    }
    __syncthreads();  // staging / column maxima free for the next tile
  }

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next kernel on the stream may begin to launch
  if (PASS == 0) {
    if (!x_row) {
      tmax_x = warp_max(tmax_x);
      if (lane == 0) atomic_absmax(p.max_x, tmax_x);
    }
    if (!w_row) {
      tmax_w = warp_max(tmax_w);
      if (lane == 0) atomic_absmax(p.max_w, tmax_w);
    }
  }
  if (!ok && tid == 0 && p.status) atomicOr(p.status, (uint32_t)HOT_STATUS_GO_DUAL);
  __syncthreads();
  if (tid == 0 && *abort_flag) {
    const uint64_t t0 = global_timer_ns();  // let bulk copies already issued land before exit
    while (global_timer_ns() - t0 < 100000ull) {
    }
  }
}

template <typename T>
constexpr int smem_bytes() { return 2 * Tile<T>::kBytes + kTC * kStagePitch + 64 + 128; }

template <typename T, int PASS, int RX, int RW, bool FAST, bool X4>
int launch_pass_as(const CUtensorMap& tmap, const DualParams& p, int grid, cudaStream_t st) {
  auto kernel = go_dual_kernel<T, PASS, RX, RW, FAST, X4>;
  static PerDeviceOnce attr_set;  // per instantiation and device
  bool have_attr = false;
  const int dev = attr_set.current(&have_attr);
  if (dev < 0) HOT_FAIL(HOT_ERR_CUDA, "go_dual_quant: cannot query the current CUDA device");
  if (!have_attr) {
    HOT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<T>()));
    attr_set.mark(dev);
  }
  if (PASS == 1) {
    // may start while the statistics pass (the launch before it on this stream) is still draining
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes<T>();
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HOT_CUDA(cudaLaunchKernelEx(&cfg, kernel, tmap, p));
  } else {
    kernel<<<grid, kThreads, smem_bytes<T>(), st>>>(tmap, p);
  }
  HOT_CUDA(cudaGetLastError());
  return HOT_OK;
}

template <typename T, int PASS, int RX, int RW>
int launch_pass(const CUtensorMap& tmap, const DualParams& p, int grid, cudaStream_t st) {
  if (p.n_o == 16 && !p.x_row && !p.w_row) {
    if (p.x_store4 || PASS == 0) return launch_pass_as<T, PASS, RX, RW, true, true>(tmap, p, grid, st);  // the statistics pass stores no codes
    return launch_pass_as<T, PASS, RX, RW, true, PASS == 1 ? false : true>(tmap, p, grid, st);
  }
  return launch_pass_as<T, PASS, RX, RW, false, true>(tmap, p, grid, st);
}

template <typename T>
int launch_dual(const void* go, int64_t ldgo, const DualParams& p, int rx, int rw, int sms, cudaStream_t st) {
  CUtensorMap tmap;
  if (int rc = make_map(&tmap, go, p.L, (int64_t)p.O * sizeof(T), ldgo * (int64_t)sizeof(T), Tile<T>::kRowBytes, kTT, 0))
    return rc;
  const int num_tiles = (p.O / kTC) * (int)((p.L + kTT - 1) / kTT);
  const int per_sm = sizeof(T) == 2 ? 3 : 1;  // resident CTAs per SM by shared memory (75 KB / 140 KB each)
  int grid = sms * per_sm;
  if (grid > num_tiles) grid = num_tiles;
  // one clear when the two abs-max regions lie close together in the caller's scratch (one launch fewer)
  const size_t nx = p.x_row ? (size_t)p.L : 1, nw = p.w_row ? (size_t)p.O : 1;
  if (p.max_w >= p.max_x + nx && (size_t)(p.max_w - p.max_x) + nw <= (1u << 18)) {
    HOT_CUDA(cudaMemsetAsync(p.max_x, 0, sizeof(uint32_t) * ((size_t)(p.max_w - p.max_x) + nw), st));
  } else {
    HOT_CUDA(cudaMemsetAsync(p.max_x, 0, sizeof(uint32_t) * nx, st));
    HOT_CUDA(cudaMemsetAsync(p.max_w, 0, sizeof(uint32_t) * nw, st));
  }
  if (int rc = launch_pass<T, 0, HOT_ROUND_NEAREST, HOT_ROUND_NEAREST>(tmap, p, grid, st)) return rc;
  const bool px = rx == HOT_ROUND_STOCH_PHILOX, pw = rw == HOT_ROUND_STOCH_PHILOX;
  if (px && pw) return launch_pass<T, 1, HOT_ROUND_STOCH_PHILOX, HOT_ROUND_STOCH_PHILOX>(tmap, p, grid, st);
  if (px) return launch_pass<T, 1, HOT_ROUND_STOCH_PHILOX, HOT_ROUND_NEAREST>(tmap, p, grid, st);
  if (pw) return launch_pass<T, 1, HOT_ROUND_NEAREST, HOT_ROUND_STOCH_PHILOX>(tmap, p, grid, st);
  return launch_pass<T, 1, HOT_ROUND_NEAREST, HOT_ROUND_NEAREST>(tmap, p, grid, st);
}

}  // namespace

int device_sm_count();

// Whether the fused kernels cover this configuration (else the caller runs the two separate ones).
bool go_dual_supported(int64_t L, int64_t O, int64_t ldgo, int dtype, int order_o, int order_l, int rank_l,
                       const int32_t* sel_l, const hot_quant_t& q_gx, const hot_quant_t& q_gw) {
  const int esz = dtype == HOT_F32 ? 4 : 2;
  if (order_l != 16 || rank_l != 8) return false;
  for (int j = 0; j < 8; ++j)
    if (sel_l[j] != kHalf16Sel[j]) return false;
  return (dtype == HOT_F32 || dtype == HOT_BF16) && order_l == 16 && rank_l == 8 && L % 32 == 0 && O % kTC == 0 &&
         O <= (1 << 24) && (ldgo * esz) % 16 == 0 && order_o >= 1 && order_o <= 64 && q_gw.storage == HOT_STORE_INT8 &&
         q_gx.rounding != HOT_ROUND_STOCH_NOISE && q_gw.rounding != HOT_ROUND_STOCH_NOISE;
}

int go_dual_quant(const void* go, int dtype, int64_t L, int64_t O, int64_t ldgo, int order_o, const int32_t* sel_l,
                  const hot_quant_t& q_gx, const hot_quant_t& q_gw, void* q_go, int64_t ld_qgo, float* s_gx, void* q_gw_t,
                  int64_t ld_qgw, float* s_gw, uint32_t* max_x, uint32_t* max_w, uint32_t* status, cudaStream_t st) {
  DualParams p;
  p.L = L;
  p.O = (int)O;
  p.n_o = order_o;
  for (int j = 0; j < 8; ++j)
    if (sel_l[j] != kHalf16Sel[j]) HOT_FAIL(HOT_ERR_UNSUPPORTED, "go_dual_quant: row selection is not the half16 preset");
  p.x_row = q_gx.scale_mode == HOT_SCALE_ROW;
  p.w_row = q_gw.scale_mode == HOT_SCALE_ROW;
  p.x_store4 = q_gx.storage == HOT_STORE_INT4;
  p.qx = make_quant_dev(q_gx);
  p.qw = make_quant_dev(q_gw);
  p.q_go = (uint8_t*)q_go;
  p.ld_qgo = ld_qgo;
  p.q_gw = (uint8_t*)q_gw_t;
  p.ld_qgw = ld_qgw;
  p.s_x = s_gx;
  p.s_w = s_gw;
  p.max_x = max_x;
  p.max_w = max_w;
  p.status = status;
  p.wait_ns = wait_limit_ns();
  const int sms = device_sm_count();
  if (sms <= 0) return HOT_ERR_CUDA;
  if (dtype == HOT_F32) return launch_dual<float>(go, ldgo, p, q_gx.rounding, q_gw.rounding, sms, st);
  return launch_dual<__nv_bfloat16>(go, ldgo, p, q_gx.rounding, q_gw.rounding, sms, st);
}

}  // namespace hot
