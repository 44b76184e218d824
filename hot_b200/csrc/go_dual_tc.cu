// grad_output (bf16) -> both quantised operands of the backward, with the two +-1 transforms run on
// the tensor cores: the Hadamard transform of order 16 along the channels (g_x side) and the
// low-rank Walsh-Hadamard projection along the tokens (g_w side, 8 lowest-sequency rows of H_16)
// are small matrix products against +-1 matrices, so a tile of grad_output that TMA laid in shared
// memory is multiplied, as it lies there, once as a K-major operand (rows = tokens) and once as an
// MN-major operand (rows = channels) by tcgen05.mma.kind::f16.  The products of bf16 values with +-1
// are exact and are summed in fp32 in tensor memory; the CUDA cores are left with what cannot be a
// matrix product: abs-max (pass 0), scaling, Philox rounding and packing (pass 1).
//
// One persistent CTA per SM walks 128-token x 128-channel tiles.  Warp roles:
//   warp 0      TMA producer: two 128-token x 64-channel boxes (128-byte swizzle) per tile
//   warp 1      allocates tensor memory and issues, from one lane, 8 MMAs (M 128 tokens, N 16, K 16
//               channels) for the channel transform and, in pass 1, 8 (M 128 channels, N 16 = two token
//               blocks x 8 kept rows, K 16 tokens) for the token projection; accumulators are
//               double-buffered.  (In pass 0 the g_w-side warps take the projection's abs-max from the
//               tile in shared memory with the butterfly of the separate kernels.)
//   warps 2-17  g_x side: a lane owns a token; each warp reads one 32-channel chunk of the lane's 128
//               transformed channels from tensor memory, quantises it and hands a 32-token box of
//               codes to the copy engine
//   warps 18-25 g_w side: a lane owns a channel; each warp reads one 32-position chunk of the lane's 64
//               projected positions, quantises it and stores it as a row piece of the transposed
//               operand the same way
//   All 24 epilogue warps work on the same tile and hand its accumulator buffer back as soon as the
//   values are in registers.  The four warps with the same chunk index wait as a group: one polls the
//   accumulator's barrier, the others sit at a named barrier.
// Measured on the ViT-B/16 fc1 gradient (12,608 x 3,072, bf16): 16 small MMAs per tile cost about as much as
// the tile's share of HBM time, which is why pass 0 issues eight; pass 1 is bound by the instruction issue of
// the rounding and packing arithmetic.
// With col_only set the kernels make the activation buffer of the forward pass (the token side alone).
//
// The fp32 sums differ from the fixed-order butterflies of row_ht_quant / col_ht_quant only where a
// sum of 16 bf16 values is not exact in fp32 (operands more than ~2^13 apart in magnitude); there the
// last bit of a transformed value may differ, and with it, rarely, a code.  The kernels therefore serve
// the nearest and Philox modes; the explicit-noise mode (bit-exact parity with the reference's
// quantisers) stays on the butterfly kernels.
//
// The layer's weight rides along (TcWeightJob): its Hadamard transform along the output features and its
// quantisation are independent of grad_output and tiny (a few MB), but as kernels of their own they cost
// three launches whose CTAs cannot share an SM with these (measured: 18 us of a 102 us fc1 backward).  Here the
// epilogue warps each take at most a few 32 x 32 pieces of the weight before their tile loop: abs-max in
// pass 0, codes in pass 1 (measured: 5 us for the 3,072 x 768 weight, most of it in pass 1, whose warps are
// the busy ones; the CTAs whose warps had pieces then simply draw fewer tiles).
// Every wait on an mbarrier is bounded in time (see gemm_i8.cu for the abort protocol).
#include "ht_device.cuh"
#include "tc.cuh"

namespace hot {
namespace {

constexpr int kTok = 128;                  // tokens per tile
constexpr int kCh = 128;                   // channels per tile
constexpr int kBoxBytes = kTok * 128;      // one TMA box: 128 tokens x 64 bf16 channels
constexpr int kStageBytes = 2 * kBoxBytes; // 32 KB
constexpr int kStages = 4;
constexpr uint32_t kBufCols = 192;         // an accumulator buffer: 128 (channel transform) + 64 (token projection) columns
constexpr uint32_t kTmemColsTc = 512;      // two buffers (384 columns), rounded up to a power of two
// Epilogue warps: the work on a tile is cut into 32-value chunks of a lane's accumulator row, one per warp,
// so that all of them work on the same tile at once: 16 on the g_x side (4 lane quarters x 4 chunks of 32
// channels) and 8 on the g_w side (4 lane quarters x 2 chunks of 32 positions).
constexpr int kRowWarps = 16, kColWarps = 8;
constexpr int kEpiWarps = kRowWarps + kColWarps;
constexpr int kThreadsTc = (2 + kEpiWarps) * 32;
constexpr int kOffOperands = kStages * kStageBytes;      // H16 | P (first block) | P (second block): 512 bytes each
constexpr int kOffStoreStage = kOffOperands + 2048;      // per epilogue warp two boxes of 32 rows x 32 bytes
constexpr int kOffBarriers = kOffStoreStage + kEpiWarps * 2048;
constexpr int kSmemTc = kOffBarriers + 512 + 1024;       // barriers and tile descriptors + slack to align the base to 1024
// Tiles are handed out at run time: the producer thread draws the next tile from a counter in global memory and
// leaves its coordinates in a ring of descriptors in shared memory, where every role reads them once the tile's
// data barrier has let it through.  A descriptor is written after the wait for its stage, i.e. when the
// epilogue of the tile six places back (four stages, two accumulator buffers) has its values in registers, so
// eight slots cannot be overrun.  After the last tile the producer writes a descriptor that says so and completes
// the stage's barrier by hand; the MMA thread passes that on through the accumulator's barrier.  A CTA that starts
// late, or not at all while another kernel holds its SM, therefore costs the others only the tiles it does not take.
constexpr int kSched = 8;

// natural row of H_16 of output slot j of the token projection (the 8 lowest-sequency rows)
__device__ constexpr int kSlotRow[8] = {0, 8, 12, 4, 6, 14, 10, 2};
constexpr int kSlotRowHost[8] = {0, 8, 12, 4, 6, 14, 10, 2};

struct TcParams {
  int64_t L;
  int O;
  int x_row, w_row;        // per-token scale on the g_x side, per-channel scale on the g_w side
  QuantDev qx, qw;
  float* s_x;              // [1] or [L]
  float* s_w;              // [1] or [O]
  uint32_t* max_x;         // [1] or [L]
  uint32_t* max_w;         // [1] or [O]
  uint32_t* status;
  uint32_t* counters;      // [2], zero before pass 0: tiles drawn in pass 0 / in pass 1
  uint64_t wait_ns;        // time limit of a device-side wait
  // the token side alone (the activation buffer of the forward pass: x -> INT8 codes of its low-rank projection,
  // transposed): no channel transform is issued and the g_x-side warps only keep the barriers' counts
  int col_only;
  // the weight that rides along (wt == nullptr: none): [O, wt_cols] bf16 -> codes [wt_cols, O], one per byte
  const uint16_t* wt;
  int64_t ld_wt, ld_qwt;
  int wt_cols;             // a multiple of 32
  int wt_philox;           // Philox rounding, else to nearest
  uint8_t* q_wt;
  float* s_wt;             // [1]
  uint32_t* max_wt;        // [1]
  QuantDev qwt;
};

// Instruction descriptor: D = F32, A = B = BF16, B K-major, A K-major or MN-major, M = 128, N = 16.
__host__ __device__ constexpr uint32_t instr_desc_bf16(bool a_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
}

// byte offset of element (n, k) of a 16 x 16 bf16 K-major operand without swizzle: 8 x 16-byte core
// matrices, the two K halves 128 bytes apart (leading offset), the two row groups 256 bytes apart (stride offset)
__device__ __forceinline__ int operand_offset(int n, int k) { return (n >> 3) * 256 + (k >> 3) * 128 + (n & 7) * 16 + (k & 7) * 2; }

__device__ __forceinline__ uint16_t pm_one_bf16(int negative) { return negative ? 0xBF80u : 0x3F80u; }

// 32 consecutive values of this lane's row of the accumulator -> K bits (RN(x * mk + ck)) of Philox rounding
__device__ __forceinline__ void kbits32(const uint32_t (&f)[32], const ScalePair& sp, uint32_t (&k)[32]) {
  const float2 mk2 = make_float2(sp.mk, sp.mk), ck2 = make_float2(sp.ck, sp.ck);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 t = __ffma2_rn(make_float2(__uint_as_float(f[2 * i]), __uint_as_float(f[2 * i + 1])), mk2, ck2);
    k[2 * i] = __float_as_uint(t.x);
    k[2 * i + 1] = __float_as_uint(t.y);
  }
}

// The 32 codes of elements e0 .. e0+31 (e0 a multiple of 16; of 32 when the codes take 4 random bits and
// `aligned32` is set, so that one Philox block serves both runs).  Output: INT4 packed (STORE4: 16 bytes in
// out[0..3]) or one code per byte (32 bytes in out[0..7]): run 0 first, within a run the stored order.
// BITS: the code width when it is known at compile time (4 or 8: everything that depends on it folds to
// immediates and the width-dependent choices disappear from the instruction stream), 0: read from q.
template <int ROUND, bool STORE4, int BITS>
__device__ __forceinline__ void quantise32(const uint32_t (&f)[32], const ScalePair& sp, const QuantDev& q, uint64_t e0,
                                           bool aligned32, uint32_t (&out)[8]) {
  const uint32_t off = BITS ? (1u << (BITS - 1)) : (uint32_t)(q.qmax + 1.0f);
  if (ROUND == HOT_ROUND_STOCH_PHILOX) {
    const bool rb4 = BITS ? BITS <= 4 : rand_bits(q.qmax) == 4;
    uint32_t k[32];
    kbits32(f, sp, k);
    uint4 b0, b1;
    if (rb4 && aligned32) {
      b0 = philox_block(q, e0 >> 5);
      b1 = b0;
    } else if (rb4) {
      b0 = philox_block(q, e0 >> 5);
      b1 = philox_block(q, (e0 + 16) >> 5);
    } else {
      b0 = philox_block(q, e0 >> 4);
      b1 = philox_block(q, (e0 >> 4) + 1);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint4 b = r ? b1 : b0;
      // rb4: which half of the block this run takes (known at compile time when both runs share an aligned block)
      const bool hi = aligned32 ? r == 1 : ((e0 + 16 * r) & 16u) != 0;
      uint32_t wa0, wa1, wb0, wb1;
      philox_run16_words(k + 16 * r, k + 16 * r + 8, rb4, rb4 ? (hi ? b.z : b.x) : b.x, rb4 ? (hi ? b.w : b.y) : b.y, b.z, b.w,
                         wa0, wa1, wb0, wb1);
      if (STORE4) {
        out[2 * r] = remove_offset(((wa0 >> 4) & 0x0F0F0F0Fu) | (wb0 & 0xF0F0F0F0u), off, 0x11111111u, 0x10u);
        out[2 * r + 1] = remove_offset(((wa1 >> 4) & 0x0F0F0F0Fu) | (wb1 & 0xF0F0F0F0u), off, 0x11111111u, 0x10u);
      } else {
        if (rb4) {
          wa0 = (wa0 >> 4) & 0x0F0F0F0Fu; wa1 = (wa1 >> 4) & 0x0F0F0F0Fu;
          wb0 = (wb0 >> 4) & 0x0F0F0F0Fu; wb1 = (wb1 >> 4) & 0x0F0F0F0Fu;
        }
        out[4 * r] = remove_offset(wa0, off, 0x01010101u, 0x100u);
        out[4 * r + 1] = remove_offset(wa1, off, 0x01010101u, 0x100u);
        out[4 * r + 2] = remove_offset(wb0, off, 0x01010101u, 0x100u);
        out[4 * r + 3] = remove_offset(wb1, off, 0x01010101u, 0x100u);
      }
    }
  } else {
    const int qmax = BITS ? (1 << (BITS - 1)) - 1 : (int)q.qmax;
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = 0u;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int c = quantise_one<HOT_ROUND_NEAREST>(__uint_as_float(f[16 * r + i]), sp, 0.0f, qmax);
        if (STORE4) out[2 * r + ((i & 7) >> 2)] |= (uint32_t)(c & 0xF) << (8 * (i & 3) + 4 * (i >> 3));
        else out[4 * r + (i >> 2)] |= (uint32_t)(c & 0xFF) << (8 * (i & 3));
      }
    }
  }
}

// The weight pieces of one epilogue warp.  A piece is 32 rows (two blocks of the order-16 transform along the
// output features) x 32 columns (lane = column, i.e. input feature); consecutive pieces go to consecutive
// CTAs, so the CTAs that run side by side read neighbouring 64-byte stretches of the same rows.  The
// butterfly is the one of col_ht_quant (stages 1, 2, 4, 8 in place), so the transformed values and the codes
// are bit-identical to that kernel's; a lane's 32 codes are one aligned run of the stored row of its column
// (element index = column * O + position), i.e. exactly one Philox block of 4-bit draws or two of 8-bit draws.
// Warp e of CTA b takes pieces e * gridDim.x + b, + kEpiWarps * gridDim.x, ...
struct WeightWalk {
  int pieces, col_groups, first, step;
};
__device__ __forceinline__ WeightWalk weight_walk(const TcParams& p, int e) {
  WeightWalk w;
  w.col_groups = p.wt_cols >> 5;
  w.pieces = (p.O >> 5) * w.col_groups;
  w.first = e * (int)gridDim.x + (int)blockIdx.x;
  w.step = kEpiWarps * (int)gridDim.x;
  return w;
}
// loads piece u and transforms it: v[16 * b + k] = row k of H_16 applied to rows 16 * b .. 16 * b + 15 of the piece
__device__ __forceinline__ void weight_piece_load(const TcParams& p, const WeightWalk& w, int u, int lane, float (&v)[32]) {
  const int rb = u / w.col_groups, c = (u - rb * w.col_groups) * 32 + lane;
  const uint16_t* src = p.wt + (int64_t)(rb * 32) * p.ld_wt + c;
#pragma unroll
  for (int r = 0; r < 32; ++r) v[r] = __uint_as_float((uint32_t)__ldg(src + (int64_t)r * p.ld_wt) << 16);
#pragma unroll
  for (int b = 0; b < 2; ++b)
#pragma unroll
    for (int h = 1; h < 16; h <<= 1)
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if ((i & h) == 0) {
          const float a = v[16 * b + i], d = v[16 * b + i + h];
          v[16 * b + i] = a + d;
          v[16 * b + i + h] = a - d;
        }
}
__device__ __forceinline__ void weight_piece_quant(const TcParams& p, const WeightWalk& w, int u, int lane, const float (&v)[32],
                                                   const ScalePair& sp) {
  const int rb = u / w.col_groups, c = (u - rb * w.col_groups) * 32 + lane;
  uint32_t f[32], out[8];
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = __float_as_uint(v[i]);
  const uint64_t e0 = (uint64_t)c * (uint64_t)p.O + (uint64_t)(rb * 32);
  if (!p.wt_philox) quantise32<HOT_ROUND_NEAREST, false, 0>(f, sp, p.qwt, e0, true, out);
  else if (p.qwt.qmax == 7.0f) quantise32<HOT_ROUND_STOCH_PHILOX, false, 4>(f, sp, p.qwt, e0, true, out);  // the usual width, folded
  else quantise32<HOT_ROUND_STOCH_PHILOX, false, 0>(f, sp, p.qwt, e0, true, out);
  uint4* dst = reinterpret_cast<uint4*>(p.q_wt + (int64_t)c * p.ld_qwt + rb * 32);
  dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
  dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
}

// PASS 0: abs-max of both transformed tensors.  PASS 1: quantise against them (RX / RW: rounding of the
// g_x / g_w side; X4: g_x codes packed INT4, else one per byte).  Pass 1 walks the tiles in the reverse
// order of pass 0, so that it starts on the part of grad_output that is most likely still in L2.
// FAST: the widths of the training configuration (4-bit codes on the g_x side, 8-bit on the g_w side) and one
// scale per tensor on both sides, folded at compile time.
template <int PASS, int RX, int RW, bool X4, bool FAST>
__global__ void __launch_bounds__(kThreadsTc, 1)
    go_dual_tc_kernel(const __grid_constant__ CUtensorMap tmap_in, const __grid_constant__ CUtensorMap tmap_qgo,
                      const __grid_constant__ CUtensorMap tmap_qgw, TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kOffBarriers);   // tile landed
  uint64_t* empty = full + kStages;                                    // the tile's MMAs retired
  uint64_t* tmem_full = empty + kStages;                               // [2] both accumulators of a tile complete
  uint64_t* tmem_empty = tmem_full + 2;                                // [2] drained by the epilogue warps
  volatile int2* sched_tile = reinterpret_cast<volatile int2*>(tmem_empty + 2);  // [kSched] (token tile, channel tile); x < 0: no more tiles
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(const_cast<int2*>(sched_tile + kSched));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool x_row = FAST ? false : p.x_row != 0, w_row = FAST ? false : p.w_row != 0;
  const int tiles_c = p.O / kCh;
  const int tiles_t = (int)((p.L + kTok - 1) / kTok);
  const int num_tiles = tiles_c * tiles_t;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], PASS == 0 ? 1 + kColWarps : 1);  // pass 0: the g_w side reads the tile itself (below)
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], PASS == 0 ? kRowWarps : kEpiWarps);  // one elected lane per warp that reads it
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tma_prefetch_desc(&tmap_in);
    if (PASS == 1) {
      tma_prefetch_desc(&tmap_qgo);
      tma_prefetch_desc(&tmap_qgw);
    }
  }
  // the three +-1 operands: H_16, and the kept rows of H_16 placed for the first / second token block of a pair
  if (threadIdx.x < 256) {
    const int n = threadIdx.x >> 4, k = threadIdx.x & 15;
    uint8_t* ops = smem + kOffOperands;
    *reinterpret_cast<uint16_t*>(ops + operand_offset(n, k)) = pm_one_bf16(__popc(n & k) & 1);
    const uint16_t pv = pm_one_bf16(__popc(kSlotRow[n & 7] & k) & 1);
    *reinterpret_cast<uint16_t*>(ops + 512 + operand_offset(n, k)) = n < 8 ? pv : (uint16_t)0;
    *reinterpret_cast<uint16_t*>(ops + 1024 + operand_offset(n, k)) = n < 8 ? (uint16_t)0 : pv;
  }
  fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
  if (warp == 1) tmem_alloc(tmem_slot, kTmemColsTc);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer (grad_out is not written by the kernel before this one: no dependency wait) ----
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      // A CTA's first tile is its own index, so that the first copy does not wait for a round trip to the counter;
      // after that the draw for the next tile is in flight while this one's waits and copies are issued (a CTA ends
      // up drawing one number more than it uses).
      int next = (int)blockIdx.x;
      for (uint32_t it = 0;; ++it, s = (s + 1 == kStages ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
        const int seq = next;
        if (seq < num_tiles) next = (int)(gridDim.x + atomicAdd(p.counters + PASS, 1u));
        if (!mbar_wait_parked(&empty[s], ph ^ 1u, abort_flag, p.wait_ns)) break;
        volatile int2* desc = sched_tile + (it % kSched);
        if (seq >= num_tiles) {
          desc->x = -1;
          mbar_arrive(&full[s]);  // no data: the phase completes on this arrival alone
          break;
        }
        const int t = PASS == 0 ? seq : num_tiles - 1 - seq;  // pass 1 takes the tiles in the reverse order of pass 0 (see above)
        const int tt = t / tiles_c, tc = t % tiles_c;
        desc->x = tt;
        desc->y = tc;
        mbar_expect_tx(&full[s], kStageBytes);  // (release: the descriptor is visible to whoever sees this phase complete)
        tma_load_2d(smem + s * kStageBytes, &tmap_in, &full[s], tc * (kCh * 2), tt * kTok);
        tma_load_2d(smem + s * kStageBytes + kBoxBytes, &tmap_in, &full[s], tc * (kCh * 2) + 128, tt * kTok);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue ----
    if (lane == 0) {
      constexpr uint32_t idesc_row = instr_desc_bf16(false), idesc_col = instr_desc_bf16(true);
      const uint32_t ops = smem_u32(smem + kOffOperands);
      const uint64_t b_h = smem_desc(ops, 128, 256, 0);
      const uint64_t b_p0 = smem_desc(ops + 512, 128, 256, 0), b_p1 = smem_desc(ops + 1024, 128, 256, 0);
      uint32_t s = 0, ph = 0;
      for (uint32_t it = 0;; ++it, s = (s + 1 == kStages ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
        const uint32_t buf = it & 1u, bph = (it >> 1) & 1u;
        if (!mbar_wait_parked(&tmem_empty[buf], bph ^ 1u, abort_flag, p.wait_ns)) break;
        if (!mbar_wait_parked(&full[s], ph, abort_flag, p.wait_ns)) break;
        if (sched_tile[it % kSched].x < 0) {
          mbar_arrive(&tmem_full[buf]);  // no more tiles: let the epilogue warps through to see it too
          break;
        }
        tc_fence_after();
        const uint32_t stage = smem_u32(smem + s * kStageBytes);
        const uint32_t d_row = tmem_base + buf * kBufCols, d_col = d_row + 128;
        // channel transform: tokens are the rows of a K-major operand (128 bytes per token, 8-token groups 1024
        // bytes apart); 16 channels = 32 bytes of K per MMA
        if (!p.col_only) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const uint64_t a = smem_desc(stage + (g >> 2) * kBoxBytes + (g & 3) * 32, 16, 1024, 2);
            umma_bf16(d_row + 16 * g, a, b_h, idesc_row, 0u);
          }
        }
        // token projection: channels are the rows of an MN-major operand (64 channels contiguous, the next 64 in the
        // second box = leading offset; 8-token groups 1024 bytes apart = stride offset); a pair of 16-token blocks per
        // 16 output columns, one block per MMA
#pragma unroll
        for (int j = 0; j < (PASS == 0 ? 0 : 4); ++j) {
          const uint64_t a0 = smem_desc(stage + (32 * j) * 128, kBoxBytes, 1024, 2);
          const uint64_t a1 = smem_desc(stage + (32 * j + 16) * 128, kBoxBytes, 1024, 2);
          umma_bf16(d_col + 16 * j, a0, b_p0, idesc_col, 0u);
          umma_bf16(d_col + 16 * j, a1, b_p1, idesc_col, 1u);
        }
        if (PASS == 0 && p.col_only) {  // nothing was issued: the two barriers take plain arrivals
          mbar_arrive(&empty[s]);
          mbar_arrive(&tmem_full[buf]);
        } else {
          umma_commit(&empty[s]);
          umma_commit(&tmem_full[buf]);
        }
      }
    }
  } else {
    // ---- epilogue: one 32-value chunk of the tile per warp ----
    const int e = warp - 2;
    const int q = warp & 3;                 // tensor-memory lane quarter this warp may read
    const bool col_side = e >= kRowWarps;
    const int chunk = col_side ? (e - kRowWarps) >> 2 : e >> 2;  // 32 channels (of 128) / 32 positions (of 64)
    uint8_t* const store_stage = smem + kOffStoreStage + e * 2048;
    uint32_t boxes = 0;
    ScalePair sp_x = scale_from_absmax(0.0f, p.qx.qmax), sp_w = scale_from_absmax(0.0f, p.qw.qmax);
    // the weight that rides along: in pass 1 this warp's first piece is loaded and transformed before the wait for
    // pass 0 (the weight is an input of the layer, complete before pass 0 began), so only the scaling waits
    WeightWalk ww = {0, 1, 0, 1};
    float wv[32];
    if (p.wt != nullptr) {
      ww = weight_walk(p, e);
      if (PASS == 1 && ww.first < ww.pieces) weight_piece_load(p, ww, ww.first, lane, wv);
    }
    if (PASS == 1) {
      // launched as a programmatic dependent of pass 0: its abs-maxima are visible once this returns
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (!x_row && !p.col_only) sp_x = scale_from_absmax(__uint_as_float(p.max_x[0]), p.qx.qmax);
      if (!w_row) sp_w = scale_from_absmax(__uint_as_float(p.max_w[0]), p.qw.qmax);
      if (blockIdx.x == 0 && warp == 2 && lane == 0) {
        if (!x_row && !p.col_only) p.s_x[0] = sp_x.s;
        if (!w_row) p.s_w[0] = sp_w.s;
      }
    }
    if (p.wt != nullptr) {
      if (PASS == 0) {
        float m = 0.0f;
        for (int u = ww.first; u < ww.pieces; u += ww.step) {
          weight_piece_load(p, ww, u, lane, wv);
          float m4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], fabsf(wv[i]));
          m = fmaxf(m, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
        }
        if (ww.first < ww.pieces) {
          m = warp_max(m);
          if (lane == 0) atomic_absmax(p.max_wt, m);
        }
      } else {
        const ScalePair sp_wt = scale_from_absmax(__uint_as_float(p.max_wt[0]), p.qwt.qmax);
        if (blockIdx.x == 0 && warp == 2 && lane == 0) p.s_wt[0] = sp_wt.s;
        for (int u = ww.first; u < ww.pieces; u += ww.step) {
          if (u != ww.first) weight_piece_load(p, ww, u, lane, wv);
          weight_piece_quant(p, ww, u, lane, wv, sp_wt);
        }
      }
    }
    float tmax = 0.0f;  // pass 0: this thread's maximum for the per-tensor scale of its side
    const int64_t out_len = p.L / 2;
    const int grp = e >> 2;  // four warps (one per lane quarter) with the same chunk index
    for (uint32_t it = 0;; ++it) {
      const uint32_t buf = it & 1u, bph = (it >> 1) & 1u;
      const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
      // The four warps of a group wait as one: the first polls the barrier of the tile's data (the accumulators; in
      // pass 0 on the g_w side the tile itself), the others sit at a named barrier, which costs them no issue slots.
      if ((e & 3) == 0)
        mbar_wait_parked(PASS == 0 && col_side ? &full[s] : &tmem_full[buf], PASS == 0 && col_side ? ph : bph, abort_flag, p.wait_ns);
      asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
      const int tt = sched_tile[it % kSched].x, tc = sched_tile[it % kSched].y;
      if (tt < 0 || *abort_flag) break;  // no more tiles, or a wait ran out somewhere (every warp of the group sees it after the barrier)
      if (p.col_only && !col_side) {
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);  // nothing of this tile is this warp's: keep the count
        continue;
      }
      if (PASS == 0 && col_side) {
        // Pass 0, g_w side: the abs-max of the token projection comes from the CUDA cores, straight from the tile in
        // shared memory (the butterfly of the separate kernels), so that the tensor core has the eight MMAs of the
        // channel transform left per tile; 16 would bound the pass, eight stay under its HBM time.  A warp takes one
        // box (64 channels: lane = channel pair, i.e. one 128-byte row per load, conflict-free under the swizzle) and
        // two 16-token blocks.
        const int cw = e - kRowWarps;
        const uint8_t* tile = smem + s * kStageBytes + (cw & 1) * kBoxBytes + (32 * (cw >> 1)) * 128 + (lane & 3) * 4;
        float cmax0 = 0.0f, cmax1 = 0.0f;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float2 u[16], ev[8];
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(tile + (16 * b + t) * 128 + (((lane >> 2) ^ (t & 7)) << 4));
            u[t] = make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
          }
          butterfly_tokens16_even(u, ev);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            cmax0 = fmaxf(cmax0, fabsf(ev[i].x));
            cmax1 = fmaxf(cmax1, fabsf(ev[i].y));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);  // this warp has read all it needs of the stage
        if (w_row) {
          const int ch = tc * kCh + (cw & 1) * 64 + 2 * lane;
          atomic_absmax(p.max_w + ch, cmax0);
          atomic_absmax(p.max_w + ch + 1, cmax1);
        } else {
          tmax = fmaxf(tmax, fmaxf(cmax0, cmax1));
        }
        continue;
      }
      tc_fence_after();
      const int64_t tok0 = (int64_t)tt * kTok;
      const int ch0 = tc * kCh;
      uint32_t f[32];
      tmem_ld32(tmem_base + buf * kBufCols + ((uint32_t)(q * 32) << 16) + (col_side ? 128u : 0u) + 32u * chunk, f);
      // the accumulator values are in registers: hand the buffer back before working on them
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      if (PASS == 0) {
        float m4[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // four chains
#pragma unroll
        for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], fabsf(__uint_as_float(f[i])));
        const float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        if (!col_side) {
          const int64_t tok = tok0 + q * 32 + lane;
          if (x_row) {
            if (tok < p.L) atomic_absmax(p.max_x + tok, m);
          } else {
            tmax = fmaxf(tmax, m);
          }
        } else {
          if (w_row) atomic_absmax(p.max_w + ch0 + q * 32 + lane, m);
          else tmax = fmaxf(tmax, m);
        }
        continue;
      }
      // ---- pass 1: quantise the chunk, stage it as 32 rows of 16 or 32 bytes, hand the box to the copy engine ----
      if (lane == 0) bulk_wait_group_read<1>();  // the store that last read this staging buffer is done with it
      __syncwarp();
      uint8_t* box = store_stage + (boxes & 1u) * 1024;
      ++boxes;
      uint32_t out[8];
      const CUtensorMap* map;
      int x, y;
      bool inside = true;
      if (!col_side) {
        const int64_t tok = tok0 + q * 32 + lane;
        const bool tok_ok = tok < p.L;
        ScalePair sp = sp_x;
        if (x_row) {
          sp = scale_from_absmax(tok_ok ? __uint_as_float(p.max_x[tok]) : 0.0f, p.qx.qmax);
          if (tc == 0 && chunk == 0 && tok_ok) p.s_x[tok] = sp.s;
        }
        quantise32<RX, X4, FAST ? 4 : 0>(f, sp, p.qx, (uint64_t)tok * (uint64_t)p.O + (uint64_t)(ch0 + 32 * chunk), true, out);
        map = &tmap_qgo;
        x = X4 ? (ch0 + 32 * chunk) / 2 : ch0 + 32 * chunk;
        y = (int)tok0 + q * 32;
        inside = tok0 + q * 32 < p.L;  // rows past the end of a partly covered box are clipped by the copy engine
        if (X4) {
          *reinterpret_cast<uint4*>(box + lane * 16) = make_uint4(out[0], out[1], out[2], out[3]);
        } else {
          *reinterpret_cast<uint4*>(box + lane * 32) = make_uint4(out[0], out[1], out[2], out[3]);
          *reinterpret_cast<uint4*>(box + lane * 32 + 16) = make_uint4(out[4], out[5], out[6], out[7]);
        }
      } else {
        const int ch = ch0 + q * 32 + lane;
        ScalePair sp = sp_w;
        if (w_row) {
          sp = scale_from_absmax(__uint_as_float(p.max_w[ch]), p.qw.qmax);
          if (tt == 0 && chunk == 0) p.s_w[ch] = sp.s;
        }
        const int64_t pos0 = tok0 / 2 + 32 * chunk;  // first stored position of the chunk within a row of the transposed operand
        quantise32<RW, false, FAST ? 8 : 0>(f, sp, p.qw, (uint64_t)ch * (uint64_t)out_len + (uint64_t)pos0, false, out);
        map = &tmap_qgw;
        x = (int)pos0;
        y = ch0 + q * 32;
        inside = pos0 < out_len;
        *reinterpret_cast<uint4*>(box + lane * 32) = make_uint4(out[0], out[1], out[2], out[3]);
        *reinterpret_cast<uint4*>(box + lane * 32 + 16) = make_uint4(out[4], out[5], out[6], out[7]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (inside) tma_store_2d(map, box, x, y);
        bulk_commit_group();  // always: the buffer rotation counts groups
      }
    }
    if (PASS == 0) {
      tmax = warp_max(tmax);
      if (lane == 0) {
        if (!col_side && !x_row && !p.col_only) atomic_absmax(p.max_x, tmax);
        if (col_side && !w_row) atomic_absmax(p.max_w, tmax);
      }
    } else if (lane == 0) {
      bulk_wait_group<0>();  // the staged boxes have left shared memory and are written
    }
  }

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next kernel on the stream may begin to launch
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemColsTc);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    if (p.status) atomicOr(p.status, (uint32_t)HOT_STATUS_GO_DUAL_TC);
    const uint64_t t0 = global_timer_ns();  // let bulk copies already issued land before exit
    while (global_timer_ns() - t0 < 100000ull) {
    }
  }
}

template <int PASS, int RX, int RW, bool X4, bool FAST>
int launch_tc_pass_as(const CUtensorMap& m_in, const CUtensorMap& m_qgo, const CUtensorMap& m_qgw, const TcParams& p, int grid,
                      cudaStream_t st) {
  auto kernel = go_dual_tc_kernel<PASS, RX, RW, X4, FAST>;
  static PerDeviceOnce attr_set;  // per instantiation and device
  bool have_attr = false;
  const int dev = attr_set.current(&have_attr);
  if (dev < 0) HOT_FAIL(HOT_ERR_CUDA, "go_dual_quant: cannot query the current CUDA device");
  if (!have_attr) {
    HOT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc));
    attr_set.mark(dev);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreadsTc);
  cfg.dynamicSmemBytes = kSmemTc;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = PASS == 1 ? 1 : 0;  // pass 1 may start while pass 0 (the launch before it on this stream) drains
  HOT_CUDA(cudaLaunchKernelEx(&cfg, kernel, m_in, m_qgo, m_qgw, p));
  HOT_CUDA(cudaGetLastError());
  return HOT_OK;
}

template <int PASS, int RX, int RW, bool X4>
int launch_tc_pass(const CUtensorMap& m_in, const CUtensorMap& m_qgo, const CUtensorMap& m_qgw, const TcParams& p, int grid,
                   cudaStream_t st) {
  const bool fast = !p.w_row && p.qw.qmax == 127.0f && (p.col_only || (!p.x_row && p.qx.qmax == 7.0f));  // (the g_x side does not run in col_only)
  if (PASS == 0) return launch_tc_pass_as<PASS, RX, RW, X4, false>(m_in, m_qgo, m_qgw, p, grid, st);  // nothing of it depends on the widths
  if (fast) return launch_tc_pass_as<PASS, RX, RW, X4, true>(m_in, m_qgo, m_qgw, p, grid, st);
  return launch_tc_pass_as<PASS, RX, RW, X4, false>(m_in, m_qgo, m_qgw, p, grid, st);
}

}  // namespace

int device_sm_count();

// Whether the tensor-core kernels cover this configuration (else the caller takes the butterfly kernels).
bool go_dual_tc_supported(int64_t L, int64_t O, int64_t ldgo, int dtype, int order_o, int order_l, int rank_l,
                          const int32_t* sel_l, const hot_quant_t& q_gx, const hot_quant_t& q_gw) {
  if (dtype != HOT_BF16 || order_o != 16 || order_l != 16 || rank_l != 8) return false;
  for (int j = 0; j < 8; ++j)
    if (sel_l[j] != kSlotRowHost[j]) return false;
  return L % 32 == 0 && L < (1ll << 31) && O % kCh == 0 && O <= (1 << 24) && (ldgo * 2) % 16 == 0 &&
         q_gw.storage == HOT_STORE_INT8 && q_gx.rounding != HOT_ROUND_STOCH_NOISE && q_gw.rounding != HOT_ROUND_STOCH_NOISE;
}

// Whether the tensor-core kernels can make the activation buffer: x [L, I] -> INT8 codes of its projection on the 8
// lowest-sequency rows of H_16 along the tokens, transposed, one scale.
bool abc_tc_supported(int64_t L, int64_t I, int64_t ldx, int dtype, int order_l, int rank_l, const int32_t* sel_l,
                      const hot_quant_t& q_x) {
  if (dtype != HOT_BF16 || order_l != 16 || rank_l != 8) return false;
  for (int j = 0; j < 8; ++j)
    if (sel_l[j] != kSlotRowHost[j]) return false;
  return L % 32 == 0 && L < (1ll << 31) && I % kCh == 0 && I <= (1 << 24) && (ldx * 2) % 16 == 0 && q_x.storage == HOT_STORE_INT8 &&
         q_x.scale_mode == HOT_SCALE_TENSOR && (q_x.rounding == HOT_ROUND_STOCH_PHILOX || q_x.rounding == HOT_ROUND_NEAREST);
}

// Whether the layer's weight [O, I] (same dtype and transform order as grad_out) can ride along.
bool tc_weight_job_supported(int64_t O, int64_t I, int64_t ldw, const hot_quant_t& q_w) {
  return I > 0 && I % 32 == 0 && I <= (1 << 24) && O % 32 == 0 && (O >> 5) * (I >> 5) <= (1ll << 30) && ldw >= I &&
         q_w.scale_mode == HOT_SCALE_TENSOR &&
         (q_w.rounding == HOT_ROUND_STOCH_PHILOX || q_w.rounding == HOT_ROUND_NEAREST) && q_w.bits >= 2 && q_w.bits <= 8;
}

int go_dual_quant_tc(const void* go, int64_t L, int64_t O, int64_t ldgo, const hot_quant_t& q_gx, const hot_quant_t& q_gw,
                     void* q_go, int64_t ld_qgo, float* s_gx, void* q_gw_t, int64_t ld_qgw, float* s_gw, uint32_t* max_x,
                     uint32_t* max_w, uint32_t* counters, size_t counter_words, uint32_t* status, cudaStream_t st,
                     const TcWeightJob* wj, bool col_only) {
  // col_only: the g_w side alone (q_go, s_gx, max_x unused and may be null; q_gx ignored apart from its validity)
  TcParams p;
  p.col_only = col_only ? 1 : 0;
  if (col_only) {
    q_go = q_gw_t;  // a valid address for the tensor map that is never stored through
    ld_qgo = ld_qgw;
    max_x = max_w;
  }
  p.counters = counters;  // two words: tiles drawn by each pass (the caller may have more words behind them cleared along)
  p.wt = nullptr;
  if (wj) {
    if (!tc_weight_job_supported(O, wj->I, wj->ldw, wj->q) || wj->ld_qw % 16 != 0 || wj->ld_qw < O || ((uintptr_t)wj->q_w) % 16 != 0 ||
        ((uintptr_t)wj->w) % 2 != 0)
      HOT_FAIL(HOT_ERR_ARG, "go_dual_quant: the weight cannot ride along (shape, pitch or quantiser)");
    p.wt = (const uint16_t*)wj->w;
    p.ld_wt = wj->ldw;
    p.ld_qwt = wj->ld_qw;
    p.wt_cols = (int)wj->I;
    p.wt_philox = wj->q.rounding == HOT_ROUND_STOCH_PHILOX;
    p.q_wt = (uint8_t*)wj->q_w;
    p.s_wt = wj->s_w;
    p.max_wt = wj->max_w;
    p.qwt = make_quant_dev(wj->q);
  }
  p.L = L;
  p.O = (int)O;
  p.x_row = !col_only && q_gx.scale_mode == HOT_SCALE_ROW;
  p.w_row = q_gw.scale_mode == HOT_SCALE_ROW;
  p.qx = make_quant_dev(q_gx);
  p.qw = make_quant_dev(q_gw);
  p.s_x = s_gx;
  p.s_w = s_gw;
  p.max_x = max_x;
  p.max_w = max_w;
  p.status = status;
  p.wait_ns = wait_limit_ns();
  const bool x4 = !col_only && q_gx.storage == HOT_STORE_INT4;
  CUtensorMap m_in, m_qgo, m_qgw;
  if (int rc = make_map(&m_in, go, L, O * 2, ldgo * 2, 128, kTok, 128)) return rc;
  if (col_only) {
    if (int rc = make_map(&m_qgo, q_go, O, L / 2, ld_qgo, 32, 32, 0)) return rc;
  } else if (int rc = make_map(&m_qgo, q_go, L, x4 ? O / 2 : O, ld_qgo, x4 ? 16 : 32, 32, 0)) {
    return rc;
  }
  if (int rc = make_map(&m_qgw, q_gw_t, O, L / 2, ld_qgw, 32, 32, 0)) return rc;
  const int sms = device_sm_count();
  if (sms <= 0) return HOT_ERR_CUDA;
  const int num_tiles = (int)(O / kCh) * (int)((L + kTok - 1) / kTok);
  const int grid = sms < num_tiles ? sms : num_tiles;
  const size_t nx = col_only ? 0 : (p.x_row ? (size_t)L : 1), nw = p.w_row ? (size_t)O : 1;
  // one clear where the scratch words lie close together (they do in every caller of this library), else one each
  struct Span {
    uint32_t* p;
    size_t n;
  } spans[4] = {{max_x, nx}, {max_w, nw}, {counters, counter_words < 2 ? (size_t)2 : counter_words}, {wj ? wj->max_w : max_x, wj ? (size_t)1 : (size_t)0}};
  uint32_t *lo = max_w, *hi = max_w;
  for (const Span& sp : spans) {
    if (sp.n == 0) continue;
    if (sp.p < lo) lo = sp.p;
    if (sp.p + sp.n > hi) hi = sp.p + sp.n;
  }
  size_t used = 0;
  for (const Span& sp : spans) used += sp.n;
  if ((size_t)(hi - lo) <= (1u << 18) || (size_t)(hi - lo) <= 2 * used) {
    HOT_CUDA(cudaMemsetAsync(lo, 0, sizeof(uint32_t) * (size_t)(hi - lo), st));
  } else {
    for (const Span& sp : spans)
      if (sp.n) HOT_CUDA(cudaMemsetAsync(sp.p, 0, sizeof(uint32_t) * sp.n, st));
  }
  if (int rc = launch_tc_pass<0, HOT_ROUND_NEAREST, HOT_ROUND_NEAREST, true>(m_in, m_qgo, m_qgw, p, grid, st)) return rc;
  const bool px = !col_only && q_gx.rounding == HOT_ROUND_STOCH_PHILOX, pw = q_gw.rounding == HOT_ROUND_STOCH_PHILOX;
  constexpr int N = HOT_ROUND_NEAREST, P = HOT_ROUND_STOCH_PHILOX;
  if (x4) {
    if (px && pw) return launch_tc_pass<1, P, P, true>(m_in, m_qgo, m_qgw, p, grid, st);
    if (px) return launch_tc_pass<1, P, N, true>(m_in, m_qgo, m_qgw, p, grid, st);
    if (pw) return launch_tc_pass<1, N, P, true>(m_in, m_qgo, m_qgw, p, grid, st);
    return launch_tc_pass<1, N, N, true>(m_in, m_qgo, m_qgw, p, grid, st);
  }
  if (px && pw) return launch_tc_pass<1, P, P, false>(m_in, m_qgo, m_qgw, p, grid, st);
  if (px) return launch_tc_pass<1, P, N, false>(m_in, m_qgo, m_qgw, p, grid, st);
  if (pw) return launch_tc_pass<1, N, P, false>(m_in, m_qgo, m_qgw, p, grid, st);
  return launch_tc_pass<1, N, N, false>(m_in, m_qgo, m_qgw, p, grid, st);
}

}  // namespace hot
