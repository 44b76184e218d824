// Integer GEMM  out[m, n] = dequant( sum_k a[m, k] * b[n, k] )  on the 5th-generation tensor
// cores: tcgen05.mma kind::i8, int32 accumulators in tensor memory, operands brought in by TMA.
//
// One persistent CTA per SM walks 128 x BN output tiles (BN chosen per problem).  Warp roles:
//   warp 0      TMA producer: per 128-byte K slab, one tiled bulk copy for A (128 rows) and one
//               for B (BN rows) into a 128B-swizzled shared-memory stage; completion on full[s]
//   warp 1      allocates tensor memory, issues 4 x (M128, N BN, K32) MMAs per stage from one
//               elected lane, releases the stage with tcgen05.commit -> empty[s]
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its 32-lane quarter), convert,
//               apply (acc * sa) * sb * post, store fp32 / bf16 / raw int32; the accumulator is
//               double-buffered in tensor memory, so this overlaps the next tile's MMAs
//   warps 6..13 (packed INT4 operands only) TMA lands the packed bytes in a raw stage and these
//               warps expand them to int8 into the swizzled stage before the MMA warp is
//               signalled (Blackwell has no 4-bit integer MMA kind)
//
// Every wait on an mbarrier is bounded in time; when a wait runs out the CTA ORs a code into
// the caller's status word, stops issuing work, frees its tensor memory and returns.
#include <type_traits>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "tc.cuh"

namespace hot {

int device_sm_count();

namespace {

constexpr int kBM = 128;
constexpr int kBK = 128;  // int8 elements (= bytes) of K per stage: one 128B swizzle span
constexpr int kUnpackThreads = 256;  // 8 warps expand packed INT4 operands

struct GemmParams {
  int M, N, K, num_kb;
  const float* sa;
  const float* sb;
  int sa_row, sb_row;  // 0: one scale; sa_row = k >= 1: one scale per k consecutive rows of A; sb_row: per row of B
  // grouped: the K axis is cut into groups of group_kb k-blocks with one scale pair each (a batch of
  // samples laid side by side along K); out = sum_g ((float)acc_g * ga[g]) * gb[g], then * post
  int group_kb;
  const float* ga;
  const float* gb;
  float post;
  void* out;
  int64_t ldo;
  int out_dtype;
  uint32_t* status;
  uint64_t wait_ns;  // time limit of a device-side wait
  int staged;  // the output qualifies for bulk tensor stores (16-byte aligned base and pitch)
  // stream-K: CTAs take equal contiguous ranges of (tile, k-block) units; a tile cut by a range
  // boundary is finished by whichever contributor arrives last
  int stream_k;
  int32_t* sk_partials;    // [2 * gridDim.x][128][BN] int32
  uint32_t* sk_counters;   // [num_tiles] k-blocks delivered so far (zero before launch; left zero)
  // rider of a dual launch: each of its (few, long) tiles is cut into `split` stretches of k-blocks that go to
  // different workers; their partial sums meet like those of a stream-K tile (sk_partials: one slot per
  // worker that holds a stretch, sk_counters: one word per rider tile).  0 or 1: whole tiles.
  int split;
};

// One stretch of k-blocks of one output tile.
struct Segment {
  int tile, kb0, kb1;
  int prob;    // 0: the kernel's main problem; 1: the rider problem (dual launch)
  int ltile;   // tile index within its problem
  int group;   // grouped mode: which group of the K axis
  bool first;  // first segment of this CTA (selects the partial slot)
};

// The sequence of segments of one CTA: whole tiles round-robin, or (stream-K) the units
// [total * cta / n, total * (cta + 1) / n) with total = num_tiles * num_kb.  Every warp role walks
// its own copy, so they agree on the sequence without communicating.
struct SegmentIter {
  bool stream_k, first;
  int tile, stride, num_tiles, num_kb;
  int group_kb, grp;
  long long u, end;
  // dual launch: a second ("rider") problem of few, long tiles shares the launch.  Worker w < riders
  // takes rider piece w first (a whole tile, or one of `split` stretches of its k-blocks); the main problem's
  // tiles are then dealt in rounds, in which the workers that hold a rider piece only join from round `lag`
  // on (lag = k-blocks of a piece / main k-blocks, rounded), so that every worker ends up with about the
  // same number of k-blocks.
  int riders, lag, rider_kb, rider_piece_kb, rider_split, round, me, nw;
  bool rider_pending;
  // worker / nworkers: this CTA (or CTA pair) among those that share the tiles
  __device__ SegmentIter(const GemmParams& p, int num_tiles_, int worker, int nworkers) {
    stream_k = p.stream_k != 0;
    first = true;
    num_tiles = num_tiles_;
    num_kb = p.num_kb;
    group_kb = p.group_kb;
    grp = 0;
    tile = worker;
    stride = nworkers;
    const long long total = (long long)num_tiles * num_kb;
    u = total * worker / nworkers;
    end = total * (worker + 1) / nworkers;
    riders = 0;
    rider_pending = false;
  }
  __device__ void add_rider(int rider_tiles, int rider_num_kb, int worker, int nworkers, int split) {
    rider_split = split < 1 ? 1 : split;
    riders = rider_tiles * rider_split;
    rider_kb = rider_num_kb;
    rider_piece_kb = (rider_num_kb + rider_split - 1) / rider_split;
    lag = (rider_piece_kb + num_kb / 2) / num_kb;
    round = 0;
    me = worker;
    nw = nworkers;
    rider_pending = worker < riders;
  }
  __device__ bool exhausted() const { return stream_k ? u >= end : tile >= num_tiles; }
  __device__ bool next(Segment& s) {
    s.first = first;
    first = false;
    s.group = 0;
    s.prob = 0;
    if (riders) {
      s.kb0 = 0;
      if (rider_pending) {
        rider_pending = false;
        s.prob = 1;
        s.ltile = me / rider_split;
        s.tile = num_tiles + s.ltile;
        s.kb0 = (me % rider_split) * rider_piece_kb;
        s.kb1 = s.kb0 + rider_piece_kb < rider_kb ? s.kb0 + rider_piece_kb : rider_kb;
        return true;
      }
      const int free_workers = nw - riders;
      for (;;) {
        const bool all = round >= lag;
        const int base = all ? lag * free_workers + (round - lag) * nw : round * free_workers;
        if (base >= num_tiles) return false;
        const int rank = all ? me : me - riders;
        ++round;
        if (rank < 0) continue;  // this worker sits the round out
        if (base + rank >= num_tiles) return false;
        s.tile = s.ltile = base + rank;
        s.kb1 = num_kb;
        return true;
      }
    }
    if (group_kb) {  // one segment per (tile, group)
      if (tile >= num_tiles) return false;
      s.tile = s.ltile = tile;
      s.group = grp;
      s.kb0 = grp * group_kb;
      s.kb1 = s.kb0 + group_kb;
      if (s.kb1 >= num_kb) {
        grp = 0;
        tile += stride;
      } else {
        ++grp;
      }
      return true;
    }
    if (!stream_k) {
      if (tile >= num_tiles) return false;
      s.tile = s.ltile = tile;
      s.kb0 = 0;
      s.kb1 = num_kb;
      tile += stride;
      return true;
    }
    if (u >= end) return false;
    s.tile = s.ltile = (int)(u / num_kb);
    s.kb0 = (int)(u - (long long)s.tile * num_kb);
    const long long left = end - u;
    const int room = num_kb - s.kb0;
    s.kb1 = s.kb0 + (int)(left < room ? left : room);
    u += s.kb1 - s.kb0;
    return true;
  }
};

// ---- CTA pairs (cta_group::2): two CTAs of a cluster run one 256 x BN tile; each holds its own 128
// rows of A and half of the rows of B in shared memory, the MMA is issued by the CTA of rank 0 and
// accumulates into the tensor memory of both ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in the CTA of the given rank
__device__ __forceinline__ uint32_t mapa_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile load into this CTA's shared memory whose completion is counted on a barrier of the pair's
// rank-0 CTA (each CTA fetches only what it holds itself)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"((uint16_t)3)
               : "memory");
}
// Shared-memory matrix descriptor: K-major operand, 128B swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (SBO), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)1u << 16;            // leading byte offset (unused for swizzled K-major), 16 B
  d |= (uint64_t)(1024u >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1u << 46;            // version
  d |= (uint64_t)2u << 61;            // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D = S32, A = B = signed 8-bit, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t instr_desc_i8(int bn, int m = kBM) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

constexpr int kSmemMax = 227 * 1024;     // what a CTA may use
constexpr int kEpiThreads = 256;          // two teams of four warps; a team covers the 128 accumulator rows
constexpr int kStoreStage = 8 * 2 * 2048;  // per epilogue warp two 32-row x 64-byte output boxes

template <int BN, bool A4, bool B4, bool PAIR = false>
struct SmemLayout {
  static_assert(!(PAIR && B4), "CTA pairs take B one code per byte");
  static constexpr int kBRows = PAIR ? BN / 2 : BN;  // rows of B this CTA holds
  static constexpr int kA = kBM * kBK;       // int8 stage of A
  static constexpr int kB = kBRows * kBK;    // int8 stage of B
  // a packed operand lands in the upper half of its own int8 stage and is expanded in place
  static constexpr int kRawA = A4 ? kBM * kBK / 2 : 0;       // bytes of packed A per stage
  static constexpr int kRawB = B4 ? kBRows * kBK / 2 : 0;
  static constexpr int kStage = kA + kB;
  static constexpr int kStagesFit = (kSmemMax - 1536 - kStoreStage) / kStage;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kOffA + kStages * kA;
  static constexpr int kOffStore = kOffB + kStages * kB;  // = bytes of the operand ring; 1024-aligned
  static constexpr int kOffBar = kOffStore + kStoreStage;
  static constexpr int kBytes = kOffBar + 512 + 1024;  // barriers + slack to align the base to 1024
  static_assert(kOffStore % 1024 == 0 && kBytes <= kSmemMax, "shared-memory plan");
  static_assert(kStages >= 2, "tile too large for shared memory");
};

// Tensor-memory columns: two accumulator buffers of BN columns, rounded up to a power of two.
__host__ __device__ constexpr uint32_t tmem_cols(int bn) { return 2 * bn <= 128 ? 128u : (2 * bn <= 256 ? 256u : 512u); }

// Packed INT4: a run of 16 codes is 8 bytes, byte j holding code j in its low nibble and code j + 8 in
// its high nibble.  Moving a nibble into the HIGH half of a byte gives 16 * code as a signed int8 with
// no sign-extension arithmetic, so operands unpacked this way are 16x too large and the accumulator
// is scaled back by 2^-4 per packed operand in the epilogue (exact: it is a multiple of 16).  With this
// layout four packed bytes turn into codes j..j+3 with one multiply (a shift, on the FMA pipe) and one
// mask, and into codes j+8..j+11 with one mask: no byte permutes.
__device__ __forceinline__ uint32_t nib_lo_x16(uint32_t w) { return (w * 16u) & 0xF0F0F0F0u; }
__device__ __forceinline__ uint32_t nib_hi_x16(uint32_t w) { return w & 0xF0F0F0F0u; }

// Expand a stage in place: its upper half holds ROWS rows x 64 packed bytes, as TMA delivered them; the
// whole stage becomes ROWS rows x 128 int8 codes in the 128-byte-swizzled layout (row r at r * 128,
// 16-byte chunk c at chunk position c ^ (r & 7)).  All unpack threads read their share into registers,
// meet at a barrier of their own (the output overwrites the packed bytes), then write.
template <int ROWS>
__device__ __forceinline__ void unpack_stage(uint8_t* stage, int tid) {
  constexpr int kItems = ROWS * 4 / kUnpackThreads;  // 16 packed bytes (32 codes = two output chunks) per item
  static_assert(ROWS * 4 % kUnpackThreads == 0, "rows per stage must be a multiple of 64");
  const uint8_t* raw = stage + ROWS * 64;
  uint4 w[kItems];
#pragma unroll
  for (int k = 0; k < kItems; ++k) w[k] = *reinterpret_cast<const uint4*>(raw + (tid + k * kUnpackThreads) * 16);
  asm volatile("bar.sync 2, %0;" ::"n"(kUnpackThreads) : "memory");
#pragma unroll
  for (int k = 0; k < kItems; ++k) {
    const int it = tid + k * kUnpackThreads;
    const int r = it >> 2, qd = it & 3;
    // (w.x, w.y) is one run of 16 codes, (w.z, w.w) the next
    const uint4 o0 = make_uint4(nib_lo_x16(w[k].x), nib_lo_x16(w[k].y), nib_hi_x16(w[k].x), nib_hi_x16(w[k].y));
    const uint4 o1 = make_uint4(nib_lo_x16(w[k].z), nib_lo_x16(w[k].w), nib_hi_x16(w[k].z), nib_hi_x16(w[k].w));
    const int c0 = qd * 2, c1 = qd * 2 + 1;
    *reinterpret_cast<uint4*>(stage + r * 128 + ((c0 ^ (r & 7)) << 4)) = o0;
    *reinterpret_cast<uint4*>(stage + r * 128 + ((c1 ^ (r & 7)) << 4)) = o1;
  }
}

// out = ((float)(acc >> S) * sa) * sb * post for two neighbouring columns: three roundings, the
// reference's order.  acc is a multiple of 2^S, so (float)acc * 2^-S (`unshift`) equals
// (float)(acc >> S) and the shift moves from the integer pipe, which this epilogue saturates first,
// to the FMA pipe.  SHIFTED: the kernel has a packed operand at all (else unshift is not applied).
template <bool SHIFTED, bool SB_ROW>
__device__ __forceinline__ float2 dequant2(const GemmParams& p, uint32_t a0, uint32_t a1, int col, float2 sa, float2 sb, float2 post,
                                           float2 unshift) {
  float2 f = make_float2((float)(int)a0, (float)(int)a1);
  if (SHIFTED) f = __fmul2_rn(f, unshift);
  if (SB_ROW) sb = make_float2(col < p.N ? p.sb[col] : 0.0f, col + 1 < p.N ? p.sb[col + 1] : 0.0f);
  return __fmul2_rn(__fmul2_rn(__fmul2_rn(f, sa), sb), post);
}

// Dequantise and store 32 consecutive accumulators of one output row:
// out = ((float)acc * sa) * sb * post  (three roundings, the reference's order), or the raw int32.
__device__ __forceinline__ void store_chunk(const GemmParams& p, int row, bool row_ok, int col0, const uint32_t (&acc)[32],
                                            float sa, float sb0) {
  if (!row_ok || col0 >= p.N) return;
  if (p.out_dtype == HOT_I32) {
    int32_t* o = reinterpret_cast<int32_t*>(p.out) + (int64_t)row * p.ldo + col0;
    if (col0 + 32 <= p.N && (p.ldo & 3) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<int4*>(o + i) = make_int4((int)acc[i], (int)acc[i + 1], (int)acc[i + 2], (int)acc[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) o[i] = (int)acc[i];
    }
    return;
  }
  float f[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float sb = p.sb_row ? ((col0 + i < p.N) ? p.sb[col0 + i] : 0.0f) : sb0;
    f[i] = __fmul_rn(__fmul_rn(__fmul_rn((float)(int)acc[i], sa), sb), p.post);
  }
  if (p.out_dtype == HOT_F32) {
    float* o = reinterpret_cast<float*>(p.out) + (int64_t)row * p.ldo + col0;
    if (col0 + 32 <= p.N && (p.ldo & 3) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) o[i] = f[i];
    }
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.ldo + col0;
    if (col0 + 32 <= p.N && (p.ldo & 7) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 w;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(f[i], f[i + 1]);
        __nv_bfloat162 t1 = __floats2bfloat162_rn(f[i + 2], f[i + 3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(f[i + 4], f[i + 5]);
        __nv_bfloat162 t3 = __floats2bfloat162_rn(f[i + 6], f[i + 7]);
        w.x = *reinterpret_cast<uint32_t*>(&t0);
        w.y = *reinterpret_cast<uint32_t*>(&t1);
        w.z = *reinterpret_cast<uint32_t*>(&t2);
        w.w = *reinterpret_cast<uint32_t*>(&t3);
        *reinterpret_cast<uint4*>(o + i) = w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) o[i] = __float2bfloat16_rn(f[i]);
    }
  }
}

// Persistent kernel: one CTA per SM walks the output tiles (n fastest, so CTAs running together
// share A rows and the whole of B in L2).  The shared-memory ring runs on across tiles; the
// accumulator is double-buffered in tensor memory so the epilogue of tile i overlaps the MMAs
// of tile i + 1.
//
// PAIR: the kernel is launched in clusters of two CTAs that work on one 256 x BN tile (see the
// cta_group::2 wrappers above).  Both CTAs run every role on their own half; what differs is that
// the operand loads of both are counted on barriers of the rank-0 CTA, whose MMA thread issues the
// instructions for the pair and signals "stage free" / "accumulator complete" into both CTAs, and that
// the rank-1 CTA reports "accumulator drained" / "operand unpacked" to the rank-0 CTA's barriers.
// GROUPED: the grouped-scale epilogue (hot_gemm_i8_grouped) as an instantiation of its own, so that the
// running sums a thread keeps across the groups of a tile share the register file with that epilogue only.
template <int BN, bool A4, bool B4, bool PAIR, bool GROUPED>
__global__ void __launch_bounds__(kEpiThreads + 64 + ((A4 || B4) ? kUnpackThreads : 0), 1)
    gemm_i8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const __grid_constant__ CUtensorMap tma_out, const __grid_constant__ CUtensorMap tma_a2,
                   const __grid_constant__ CUtensorMap tma_b2, const __grid_constant__ CUtensorMap tma_out2, GemmParams p,
                   GemmParams p2) {
  // p2 (p2.M > 0): the rider problem of a dual launch, INT8 x INT8 with the same tile width; its A
  // operand goes straight into the int8 stage even in the kernel built for a packed main operand
  using L = SmemLayout<BN, A4, B4, PAIR>;
  constexpr int STAGES = L::kStages;
  constexpr bool kUnpack = A4 || B4;
  constexpr uint32_t kTmemCols = tmem_cols(BN);
  constexpr uint32_t kBufStride = kTmemCols / 2;
  constexpr int kShift = (A4 ? 4 : 0) + (B4 ? 4 : 0);
  constexpr bool kGrouped = GROUPED;
  static_assert(!GROUPED || (!kUnpack && !PAIR), "the grouped-scale epilogue takes INT8 operands on single CTAs");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem + L::kOffA;
  uint8_t* sB = smem + L::kOffB;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kOffBar);  // TMA landed
  uint64_t* empty = full + STAGES;                                   // MMAs of the stage retired
  uint64_t* ready = empty + STAGES;                                  // unpacked (INT4 operands only)
  uint64_t* tmem_full = ready + STAGES;                              // [2] accumulator complete
  uint64_t* tmem_empty = tmem_full + 2;                              // [2] accumulator drained
  uint64_t* fix_bar = tmem_empty + 2;                                // stream-K fix-up copies landed
  uint64_t* full_a = fix_bar + 1;                                    // PAIR with packed A: this CTA's packed A landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(full_a + STAGES);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  // warps 0-7: epilogue; INT4 operands: warps 8-15 unpack; then one producer warp and one MMA warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kProducerWarp = (kEpiThreads + (kUnpack ? kUnpackThreads : 0)) / 32, kMmaWarp = kProducerWarp + 1;
  constexpr int kTileM = PAIR ? 2 * kBM : kBM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = ((p.M + kTileM - 1) / kTileM) * n_tiles;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;          // 0: the CTA that issues the pair's MMAs
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int nworkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // arrivals per phase: per thread in a single CTA; one elected lane per warp of both CTAs in a pair
  constexpr uint32_t kDrainArrivals = PAIR ? 2 * (kEpiThreads / 32) : kEpiThreads;
  constexpr uint32_t kUnpackArrivals = PAIR ? 2 * (kUnpackThreads / 32) : kUnpackThreads;
  const int n_tiles2 = (p2.N + BN - 1) / BN;                       // rider problem (dual launch)
  const int rider_tiles = p2.M > 0 ? ((p2.M + kBM - 1) / kBM) * n_tiles2 : 0;
  auto make_iter = [&]() {
    SegmentIter it(p, num_tiles, worker, nworkers);
    if (rider_tiles) it.add_rider(rider_tiles, p2.num_kb, worker, nworkers, p2.split);
    return it;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&ready[s], kUnpackArrivals);
      mbar_init(&full_a[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], kDrainArrivals);
    }
    mbar_init(fix_bar, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (p.staged) tma_prefetch_desc(&tma_out);
    if (rider_tiles) {
      tma_prefetch_desc(&tma_a2);
      tma_prefetch_desc(&tma_b2);
      if (p2.staged) tma_prefetch_desc(&tma_out2);
    }
  }
  if (warp == kMmaWarp) {
    if (PAIR) tmem_alloc_pair(tmem_slot, kTmemCols);
    else tmem_alloc(tmem_slot, kTmemCols);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  // Launched as a programmatic dependent of the kernel before it on the stream: the set-up above ran
  // while that kernel drained; its results (the operands, the scales) are visible once this returns.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      constexpr uint32_t kTx = (A4 ? L::kRawA : L::kA) + (B4 ? L::kRawB : L::kB);
      uint32_t s = 0, ph = 0;  // ring slot and phase, running on across tiles
      bool ok = true;
      SegmentIter iter = make_iter();
      Segment seg;
      const uint32_t full0 = PAIR ? mapa_rank(smem_u32(full), 0) : 0u;  // full[] of the rank-0 CTA
      while (ok && iter.next(seg)) {
        const int nt = seg.prob ? n_tiles2 : n_tiles;
        const int m0 = (seg.ltile / nt) * kTileM + (int)rank * kBM, n0 = (seg.ltile % nt) * BN;
        for (int kb = seg.kb0; kb < seg.kb1; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
          ok = mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.wait_ns);
          if (!ok) break;
          if (seg.prob) {  // rider: both operands one code per byte
            mbar_expect_tx(&full[s], L::kA + L::kB);
            tma_load_2d(sA + s * L::kA, &tma_a2, &full[s], kb * kBK, m0);
            tma_load_2d(sB + s * L::kB, &tma_b2, &full[s], kb * kBK, n0);
            continue;
          }
          if (PAIR) {
            // rank 0 announces the bytes of both CTAs; each CTA loads its rows of A and its half of B
            if (rank == 0) mbar_expect_tx(&full[s], 2u * ((A4 ? 0u : (uint32_t)L::kA) + (uint32_t)L::kB));
            if (A4) {
              mbar_expect_tx(&full_a[s], L::kRawA);
              tma_load_2d(sA + s * L::kA + L::kRawA, &tma_a, &full_a[s], kb * (kBK / 2), m0);
            } else {
              tma_load_2d_pair(sA + s * L::kA, &tma_a, full0 + 8u * s, kb * kBK, m0);
            }
            tma_load_2d_pair(sB + s * L::kB, &tma_b, full0 + 8u * s, kb * kBK, n0 + (int)rank * (BN / 2));
            continue;
          }
          mbar_expect_tx(&full[s], kTx);
          if (A4) tma_load_2d(sA + s * L::kA + L::kRawA, &tma_a, &full[s], kb * (kBK / 2), m0);
          else tma_load_2d(sA + s * L::kA, &tma_a, &full[s], kb * kBK, m0);
          if (B4) tma_load_2d(sB + s * L::kB + L::kRawB, &tma_b, &full[s], kb * (kBK / 2), n0);
          else tma_load_2d(sB + s * L::kB, &tma_b, &full[s], kb * kBK, n0);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instr_desc_i8(BN, kTileM);
      uint32_t s = 0, ph = 0, it = 0;
      bool ok = true;
      SegmentIter iter = make_iter();
      Segment seg;
      // shared-memory descriptors: the high word is the same for every operand slab, the low word is
      // (address >> 4) | leading-offset field and moves by 2 per 32-byte K step
      const uint32_t desc_hi = (uint32_t)(smem_desc_sw128(0) >> 32);
      const uint32_t a_lo0 = (uint32_t)smem_desc_sw128(smem_u32(sA)), b_lo0 = (uint32_t)smem_desc_sw128(smem_u32(sB));
      for (; ok && iter.next(seg); ++it) {
        const uint32_t buf = it & 1u, bph = (it >> 1) & 1u;
        ok = mbar_wait<PAIR>(&tmem_empty[buf], bph ^ 1u, abort_flag, p.wait_ns);  // epilogue (of both CTAs) drained this buffer
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kBufStride;
        for (int kb = seg.kb0; kb < seg.kb1; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
          ok = kUnpack ? mbar_wait<PAIR>(&ready[s], ph, abort_flag, p.wait_ns) : mbar_wait(&full[s], ph, abort_flag, p.wait_ns);
          if (ok && PAIR && kUnpack) ok = mbar_wait(&full[s], ph, abort_flag, p.wait_ns);  // B landed in both CTAs
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * (uint32_t)(L::kA >> 4), b_lo = b_lo0 + s * (uint32_t)(L::kB >> 4);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 32; ++k4) {
            const uint64_t ad = ((uint64_t)desc_hi << 32) | (a_lo + 2u * k4), bd = ((uint64_t)desc_hi << 32) | (b_lo + 2u * k4);
            if (PAIR) umma_i8_pair(d_tmem, ad, bd, idesc, (kb > seg.kb0 || k4 > 0) ? 1u : 0u);
            else umma_i8(d_tmem, ad, bd, idesc, (kb > seg.kb0 || k4 > 0) ? 1u : 0u);
          }
          if (PAIR) umma_commit_pair(&empty[s]);
          else umma_commit(&empty[s]);
        }
        if (ok) {
          if (PAIR) umma_commit_pair(&tmem_full[buf]);
          else umma_commit(&tmem_full[buf]);
        }
      }
    }
  } else if (warp < kEpiThreads / 32) {
    // ---- epilogue warps: team 0 takes the even output boxes of a tile, team 1 the odd ones ----
    // With the unpack warps in the CTA every thread starts with few registers; the unpack warp groups
    // give some back and the two epilogue warp groups take them.
    if (kUnpack) asm volatile("setmaxnreg.inc.sync.aligned.u32 152;" ::: "memory");
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    const int team = warp >> 2;
    // the problem the current segment belongs to (the rider of a dual launch has its own output, scales
    // and no INT4 shift), and what follows from it
    const GemmParams* cur = &p;
    const CUtensorMap* omap = &tma_out;
    bool raw = false, out16 = false;  // raw accumulators wanted (no scales to read); 16-bit output
    float sb0 = 0.0f;
    int shift = kShift;
    auto select_problem = [&](int prob) {
      cur = prob ? &p2 : &p;
      omap = prob ? &tma_out2 : &tma_out;
      raw = cur->out_dtype == HOT_I32;
      out16 = cur->out_dtype == HOT_BF16;
      sb0 = (cur->sb_row || raw || cur->group_kb) ? 0.0f : cur->sb[0];
      shift = prob ? 0 : kShift;
    };
    select_problem(0);
    __shared__ uint32_t s_finisher;
    uint32_t it = 0;
    bool ok = true;
    SegmentIter iter = make_iter();
    Segment seg;
    // Output path: a thread holds one row of the accumulator, so stores from registers would touch 32
    // lines per instruction.  Instead each warp lays 32 rows x 64 bytes out in a swizzled shared-memory
    // box (two boxes per warp, so that a bulk tensor store is in flight while the next box fills) and
    // one lane hands it to the copy engine, which clips rows and columns past the matrix.
    uint8_t* const store_stage = smem + L::kOffStore + warp * 4096;
    uint32_t boxes = 0;  // boxes filled by this warp so far (selects the buffer)
    float run[kGrouped ? BN / 64 : 1][32];  // grouped mode only
    auto owns = [&](int c) { return (c & 1) == team; };  // chunk c is this team's
    const uint32_t drained0 = PAIR ? mapa_rank(smem_u32(tmem_empty), 0) : 0u;  // tmem_empty[] of the rank-0 CTA
    // this thread has read all it needs of accumulator buffer `b`
    auto release_acc = [&](uint32_t b) {
      tc_fence_before();
      if (PAIR) {
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(drained0 + 8u * b);
      } else {
        mbar_arrive(&tmem_empty[b]);
      }
    };
    int m0 = 0, n0 = 0, row = 0;
    bool row_ok = false;
    float sa = 0.0f;
    // four 16-byte pieces of this lane's row of a box: the piece index is swizzled like the tensor map
    auto put = [&](uint8_t* box, int j, uint4 v) {
      *reinterpret_cast<uint4*>(box + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = v;
    };
    auto open_box = [&]() -> uint8_t* {
      if (lane == 0) bulk_wait_group_read<1>();  // the store that last read this buffer is done with it
      __syncwarp();
      return store_stage + (boxes & 1u) * 2048;
    };
    auto close_box = [&](uint8_t* box, int col) {  // col: first column of the box
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int y = m0 + q * 32;
        if (col < cur->N && y < cur->M) tma_store_2d(omap, box, col << (out16 ? 1 : 2), y);
        bulk_commit_group();  // always: the buffer rotation counts groups
      }
      ++boxes;
    };
    // 32 finished values of this lane's row, columns col0 .. col0 + 31; val(i) gives columns i, i + 1
    auto store_pairs = [&](int col0, auto&& val) {
      if (out16) {
        uint8_t* box = open_box();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f = val(8 * j + 2 * k);
            __nv_bfloat162 t = __floats2bfloat162_rn(f.x, f.y);
            w[k] = *reinterpret_cast<uint32_t*>(&t);
          }
          put(box, j, make_uint4(w[0], w[1], w[2], w[3]));
        }
        close_box(box, col0);
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint8_t* box = open_box();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f0 = val(16 * h + 4 * j), f1 = val(16 * h + 4 * j + 2);
            put(box, j, make_uint4(__float_as_uint(f0.x), __float_as_uint(f0.y), __float_as_uint(f1.x), __float_as_uint(f1.y)));
          }
          close_box(box, col0 + 16 * h);
        }
      }
    };
    // chunk c (32 columns) of the current tile, ascending; acc = accumulators before the INT4 shift
    auto emit = [&](int c, uint32_t (&acc)[32]) {
      if (!cur->staged) {
        if (kShift) {
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = (uint32_t)((int)acc[i] >> shift);
        }
        store_chunk(*cur, row, row_ok, n0 + c * 32, acc, sa, sb0);
        return;
      }
      const int col0 = n0 + c * 32;
      const float2 sa2 = make_float2(sa, sa), sb2 = make_float2(sb0, sb0), post2 = make_float2(cur->post, cur->post);
      const float us = shift ? 1.0f / (float)(1 << kShift) : 1.0f;
      const float2 unshift = make_float2(us, us);
      if (raw) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint8_t* box = open_box();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = 16 * h + 4 * j;
            put(box, j, make_uint4((uint32_t)((int)acc[i] >> shift), (uint32_t)((int)acc[i + 1] >> shift),
                                   (uint32_t)((int)acc[i + 2] >> shift), (uint32_t)((int)acc[i + 3] >> shift)));
          }
          close_box(box, col0 + 16 * h);
        }
      } else if (cur->sb_row) {  // one instance per scale layout, so the choice is not made per element
        store_pairs(col0, [&](int i) { return dequant2<kShift != 0, true>(*cur, acc[i], acc[i + 1], col0 + i, sa2, sb2, post2, unshift); });
      } else {
        store_pairs(col0, [&](int i) { return dequant2<kShift != 0, false>(*cur, acc[i], acc[i + 1], col0 + i, sa2, sb2, post2, unshift); });
      }
    };
    for (; ok && iter.next(seg); ++it) {
      select_problem(seg.prob);
      const GemmParams& p = *cur;  // from here on `p` is the segment's problem
      const int nt = seg.prob ? n_tiles2 : n_tiles;
      m0 = (seg.ltile / nt) * kTileM + (int)rank * kBM;
      n0 = (seg.ltile % nt) * BN;
      const uint32_t buf = it & 1u, bph = (it >> 1) & 1u;
      const int row_loc = q * 32 + lane;
      row = m0 + row_loc;
      row_ok = row < p.M;
      sa = (row_ok && !raw && !p.group_kb) ? (p.sa_row ? p.sa[row / p.sa_row] : p.sa[0]) : 0.0f;
      const bool whole = seg.kb0 == 0 && seg.kb1 == p.num_kb;
      // partial slot: [chunk of 32 columns][group of 4 columns][row][4] int32, so that a warp's rows are contiguous
      // (a stretch of a rider tile: the slot of this worker)
      int32_t* my_slot = p.sk_partials + (size_t)(seg.prob ? worker : 2 * blockIdx.x + (seg.first ? 0 : 1)) * kBM * BN + row_loc * 4;
      ok = mbar_wait(&tmem_full[buf], bph, abort_flag, p.wait_ns);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + buf * kBufStride + ((uint32_t)(q * 32) << 16);
      if constexpr (kGrouped) {
        // running fp32 sums of this team's chunks live in registers across the groups of a tile
        // sa_row: one scale per (group, row) of A instead of one per group
        const float ga = p.sa_row ? (row_ok ? p.ga[(size_t)seg.group * (size_t)p.M + (size_t)row] : 0.0f) : p.ga[seg.group];
        const float gb = p.gb[seg.group];
#pragma unroll
        for (int k = 0; k < BN / 64; ++k) {
          uint32_t acc[32];
          tmem_ld32(t_addr + (uint32_t)((2 * k + team) * 32), acc);
          if (k == BN / 64 - 1) release_acc(buf);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = __fmul_rn(__fmul_rn((float)(int)acc[i], ga), gb);
            run[k][i] = seg.kb0 == 0 ? v : __fadd_rn(run[k][i], v);
          }
        }
        if (seg.kb1 >= p.num_kb) {
          const float2 post2 = make_float2(p.post, p.post);
#pragma unroll
          for (int k = 0; k < BN / 64; ++k)
            store_pairs(n0 + (2 * k + team) * 32, [&](int i) { return __fmul2_rn(make_float2(run[k][i], run[k][i + 1]), post2); });
        }
        continue;
      }
      int c_last = BN / 32 - 1;  // last chunk this team reads
      while (c_last >= 0 && !owns(c_last)) --c_last;
      if (c_last < 0) release_acc(buf);
#pragma unroll 1
      for (int c = 0; c <= c_last; ++c) {
        if (!owns(c)) continue;
        uint32_t acc[32];
        tmem_ld32(t_addr + (uint32_t)(c * 32), acc);
        if (c == c_last) release_acc(buf);  // everything this thread needs of the buffer is in registers
        if (whole) {
          emit(c, acc);
        } else {
          // partial sum of a tile shared with other CTAs: park the accumulators as they are
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<int4*>(my_slot + c * (32 * kBM) + (i >> 2) * (4 * kBM)) =
                make_int4((int)acc[i], (int)acc[i + 1], (int)acc[i + 2], (int)acc[i + 3]);
        }
      }
      if (!whole) {
        // publish, count the k-blocks delivered for this tile; whoever completes the count adds up
        // every contributor's partial (its own included) and writes the tile
        asm volatile("fence.proxy.async.global;" ::: "memory");  // the finisher may read it with bulk copies
        __threadfence();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (threadIdx.x == 0) {
          const uint32_t mine = (uint32_t)(seg.kb1 - seg.kb0);
          uint32_t* counter = p.sk_counters + (seg.prob ? seg.ltile : seg.tile);
          const uint32_t before = atomicAdd(counter, mine);
          s_finisher = (before + mine == (uint32_t)p.num_kb) ? 1u : 0u;
          if (s_finisher) *counter = 0u;  // leave the counters as they were found
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (s_finisher) {
          __threadfence();
          const long long total = (long long)num_tiles * p.num_kb;
          const long long t_beg = (long long)seg.tile * p.num_kb, t_end = t_beg + p.num_kb;
          const long long G = gridDim.x;
          // contributors: the CTAs whose unit range meets [t_beg, t_end); for a rider tile the workers
          // that hold its stretches
          long long c_lo = seg.prob ? (long long)seg.ltile * p.split : t_beg * G / total;
          long long c_hi = c_lo;
          if (seg.prob) {
            c_hi = c_lo + p.split - 1;
          } else {
            while (c_lo + 1 < G && total * (c_lo + 1) / G <= t_beg) ++c_lo;
            while (c_lo > 0 && total * c_lo / G > t_beg) --c_lo;
            c_hi = c_lo;
            while (c_hi + 1 < G && total * (c_hi + 1) / G < t_end) ++c_hi;
          }
          const int ncontrib = (int)(c_hi - c_lo + 1);
          const bool rider_seg = seg.prob != 0;
          auto slot_of = [&](long long cta) {
            if (rider_seg) return p.sk_partials + (size_t)cta * kBM * BN;
            const bool cta_first = total * cta / G >= t_beg;  // its range starts inside this tile
            return p.sk_partials + (size_t)(2 * cta + (cta_first ? 0 : 1)) * kBM * BN;
          };
          // Fast path: this was the CTA's last segment, so the operand ring is idle; bulk copies bring
          // the partials of a group of chunks into it at full bandwidth and the sum reads shared memory.
          const int group = (!rider_seg && iter.exhausted()) ? L::kOffStore / (ncontrib * 32 * kBM * 4) : 0;
          if (group >= 1) {
            uint32_t fph = 0;
            for (int c0 = 0; c0 < BN / 32; c0 += group) {
              const int ng = (BN / 32 - c0) < group ? (BN / 32 - c0) : group;
              asm volatile("bar.sync 1, 256;" ::: "memory");  // the previous group has been read
              if (threadIdx.x == 0) {
                asm volatile("fence.proxy.async;" ::: "memory");
                mbar_expect_tx(fix_bar, (uint32_t)(ncontrib * ng * 32 * kBM * 4));
                for (int k = 0; k < ncontrib; ++k)
                  for (int g = 0; g < ng; ++g)
                    bulk_load(smem + (size_t)(k * ng + g) * (32 * kBM * 4), slot_of(c_lo + k) + (size_t)(c0 + g) * (32 * kBM), 32 * kBM * 4, fix_bar);
              }
              if (!mbar_wait(fix_bar, fph, abort_flag, p.wait_ns)) break;
              fph ^= 1u;
              for (int g = 0; g < ng; ++g) {
                if (!owns(c0 + g)) continue;
                int sum[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) sum[i] = 0;
                for (int k = 0; k < ncontrib; ++k) {
                  const int4* src = reinterpret_cast<const int4*>(smem + (size_t)(k * ng + g) * (32 * kBM * 4)) + row_loc;
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const int4 v = src[i * kBM];
                    sum[4 * i] += v.x; sum[4 * i + 1] += v.y; sum[4 * i + 2] += v.z; sum[4 * i + 3] += v.w;
                  }
                }
                uint32_t acc[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = (uint32_t)sum[i];
                emit(c0 + g, acc);
              }
            }
          } else {
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              if (!owns(c)) continue;
              int sum[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) sum[i] = 0;
              for (int k = 0; k < ncontrib; ++k) {
                const int4* src = reinterpret_cast<const int4*>(slot_of(c_lo + k) + (size_t)c * (32 * kBM)) + row_loc;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const int4 v = __ldcg(src + i * kBM);
                  sum[4 * i] += v.x; sum[4 * i + 1] += v.y; sum[4 * i + 2] += v.z; sum[4 * i + 3] += v.w;
                }
              }
              uint32_t acc[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) acc[i] = (uint32_t)sum[i];
              emit(c, acc);
            }
          }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");  // s_finisher is reused by the next segment
      }
    }
    if (lane == 0) bulk_wait_group<0>();  // the staged boxes have left shared memory and are written
  } else if (kUnpack && warp < kProducerWarp) {
    // ---- unpack warps (INT4 operands): raw stage -> swizzled int8 stage ----
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
    const int utid = threadIdx.x - kEpiThreads;
    const uint32_t ready0 = PAIR ? mapa_rank(smem_u32(ready), 0) : 0u;  // ready[] of the rank-0 CTA
    uint32_t s = 0, ph = 0;
    bool ok = true;
    SegmentIter iter = make_iter();
    Segment seg;
    while (ok && iter.next(seg)) {
      for (int kb = seg.kb0; kb < seg.kb1; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
        ok = mbar_wait(PAIR ? &full_a[s] : &full[s], ph, abort_flag, p.wait_ns);
        if (!ok) break;
        if constexpr (A4) {
          if (!seg.prob) unpack_stage<kBM>(sA + s * L::kA, utid);
        }
        if constexpr (B4) {
          if (!seg.prob) unpack_stage<L::kBRows>(sB + s * L::kB, utid);
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core (async proxy)
        if (PAIR) {
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(ready0 + 8u * s);
        } else {
          mbar_arrive(&ready[s]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // neither CTA leaves, or frees tensor memory, while the other may still use it
  if (warp == kMmaWarp) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    if (p.status) atomicOr(p.status, (uint32_t)HOT_STATUS_GEMM);
    // bulk copies issued before the abort land within microseconds; give them time before the
    // shared memory of this CTA is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 100000ull) {
    }
  }
}

// ---- host side ---------------------------------------------------------------------------
struct Plan {
  int bn;
  bool stream_k;
  unsigned grid;
  bool pair = false;  // clusters of two CTAs per 256 x bn tile
  double cost = 0.0;  // the model's estimate for this plan (k-block cost units)
};

// The second problem of a dual launch (INT8 x INT8, one code per byte on both sides).
struct Rider {
  const void* a;
  int64_t lda;
  const void* b;
  int64_t ldb;
  GemmParams p;
};

template <int BN, bool A4, bool B4, bool PAIR = false, bool GROUPED = false>
int launch_gemm(const void* a, int64_t lda, const void* b, int64_t ldb, const GemmParams& p, const Plan& plan, cudaStream_t st,
                const Rider* rider = nullptr) {
  using L = SmemLayout<BN, A4, B4, PAIR>;
  CUtensorMap ma, mb;
  int rc;
  if (A4) rc = make_map(&ma, a, p.M, (p.K + 15) / 16 * 8, lda, kBK / 2, kBM, 0);  // whole runs of 16 codes
  else rc = make_map(&ma, a, p.M, p.K, lda, kBK, kBM, 128);
  if (rc) return rc;
  if (B4) rc = make_map(&mb, b, p.N, (p.K + 15) / 16 * 8, ldb, kBK / 2, L::kBRows, 0);
  else rc = make_map(&mb, b, p.N, p.K, ldb, kBK, L::kBRows, 128);
  if (rc) return rc;
  // output as a byte matrix for the bulk tensor stores; otherwise the epilogue stores from registers
  const int64_t esz = p.out_dtype == HOT_BF16 ? 2 : 4;
  GemmParams pp = p;
  pp.staged = (reinterpret_cast<uintptr_t>(p.out) % 16 == 0 && (p.ldo * esz) % 16 == 0) ? 1 : 0;
  CUtensorMap mo = ma;
  if (pp.staged) {
    rc = make_map(&mo, p.out, p.M, (int64_t)p.N * esz, p.ldo * esz, 64, 32, 64);
    if (rc) return rc;
  }
  GemmParams p2 = {};  // M = 0: no rider
  CUtensorMap ma2 = ma, mb2 = mb, mo2 = mo;
  if (rider) {
    p2 = rider->p;
    rc = make_map(&ma2, rider->a, p2.M, p2.K, rider->lda, kBK, kBM, 128);
    if (rc) return rc;
    rc = make_map(&mb2, rider->b, p2.N, p2.K, rider->ldb, kBK, L::kBRows, 128);
    if (rc) return rc;
    const int64_t esz2 = p2.out_dtype == HOT_BF16 ? 2 : 4;
    p2.staged = (reinterpret_cast<uintptr_t>(p2.out) % 16 == 0 && (p2.ldo * esz2) % 16 == 0) ? 1 : 0;
    if (p2.staged) {
      rc = make_map(&mo2, p2.out, p2.M, (int64_t)p2.N * esz2, p2.ldo * esz2, 64, 32, 64);
      if (rc) return rc;
    }
  }
  auto kernel = gemm_i8_kernel<BN, A4, B4, PAIR, GROUPED>;
  static PerDeviceOnce attr_set;  // per instantiation and device
  bool have_attr = false;
  const int dev = attr_set.current(&have_attr);
  if (dev < 0) HOT_FAIL(HOT_ERR_CUDA, "gemm_i8: cannot query the current CUDA device");
  if (!have_attr) {
    HOT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
    if (A4 || B4) {
      // the register hand-over (unpack warp groups 96 -> 40, epilogue warp groups 96 -> 152) only balances
      // when the kernel starts with at least 96 registers per thread
      cudaFuncAttributes fa;
      HOT_CUDA(cudaFuncGetAttributes(&fa, kernel));
      if (fa.numRegs < 96) HOT_FAIL(HOT_ERR_UNSUPPORTED, "gemm_i8: kernel built with %d registers per thread, 96 expected", fa.numRegs);
    }
    attr_set.mark(dev);
  }
  constexpr unsigned kThreads = kEpiThreads + 64 + ((A4 || B4) ? kUnpackThreads : 0);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan.grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = L::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while its predecessor drains
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.numAttrs = 1;
  if (PAIR) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  HOT_CUDA(cudaLaunchKernelEx(&cfg, kernel, ma, mb, mo, ma2, mb2, mo2, pp, p2));
  HOT_CUDA(cudaGetLastError());
  return HOT_OK;
}

inline int64_t tiles_for(int M, int N, int bn) { return (int64_t)((M + kBM - 1) / kBM) * ((N + bn - 1) / bn); }
inline size_t sk_bytes(int sms, int bn, int64_t tiles) {
  return (size_t)2 * sms * kBM * bn * sizeof(int32_t) + (size_t)((tiles + 63) / 64 * 64) * sizeof(uint32_t);
}

// Tile width and schedule.  Measured on B200, the time per 128-byte k-block of a CTA grows only
// mildly with the tile width (~ bn + 400), so what counts is how many k-blocks the busiest CTA
// runs: whole tiles in waves, or (given a workspace) equal shares of all k-blocks with the cut
// tiles summed up by their last contributor (it reads every contributor's 128 x bn int32 partial
// through bulk copies into the idle operand ring).  Measured, that costs ~14 us + ~3.5 us per
// contributor at bn = 256, charged below in k-block equivalents, so stream-K is picked only for
// few-tile, very-long-K problems.
Plan make_plan(int M, int N, int num_kb, int sms, size_t ws_bytes, bool allow_pair, bool packed) {
  const int cands[4] = {256, 192, 128, 64};
  Plan best{128, false, 1};
  double best_cost = -1.0;
  // HOT_GEMM_SCHEDULE=streamk forces the stream-K schedule wherever it is possible (tests, tuning)
  const char* env = getenv("HOT_GEMM_SCHEDULE");
  const bool force_sk = env && env[0] == 's';
  // HOT_GEMM_PAIR=0 never uses CTA pairs, =1 always does where the operands allow
  const char* penv = getenv("HOT_GEMM_PAIR");
  const int pair_mode = !allow_pair ? 0 : (penv ? (penv[0] == '1' ? 2 : (penv[0] == '0' ? 0 : 1)) : 1);
  for (int bn : cands) {
    const int64_t tiles = tiles_for(M, N, bn);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double per_kb = bn + 400.0;
    const double dp = (double)waves * num_kb * per_kb;
    if (pair_mode != 2 && (best_cost < 0 || dp < best_cost)) {
      best_cost = dp;
      best = Plan{bn, false, (unsigned)(tiles < sms ? tiles : sms)};
    }
    if (pair_mode != 0) {
      // A pair of CTAs per 256 x bn tile: each CTA holds half of B.  Measured on B200 (int8 x int8): 8 % faster
      // than single CTAs at 16384 x 4096 x 11008 (3.18 POP/s), where a CTA runs a dozen long tiles, and
      // 4-16 % slower at ViT sizes (the hand-shakes between the two CTAs cost more per tile than the
      // halved B traffic saves); with a packed INT4 operand the partner's "unpacked" signal crosses
      // the cluster every k-block and the pair is twice as slow.  So pairs are taken for wide tiles of
      // long, many-tile problems with one-byte codes only, unless forced.
      const int64_t ptiles = (int64_t)((M + 2 * kBM - 1) / (2 * kBM)) * ((N + bn - 1) / bn);
      const int64_t pairs = sms / 2;
      const int64_t pwaves = (ptiles + pairs - 1) / pairs;
      const bool pays = !packed && bn == 256 && num_kb >= 64 && ptiles >= 4 * pairs;
      const double pc = (pair_mode == 2 || pays) ? (double)pwaves * num_kb * 0.92 * per_kb : 1e300;
      if (best_cost < 0 || pc < best_cost) {
        best_cost = pc;
        best = Plan{bn, false, (unsigned)(2 * (ptiles < pairs ? ptiles : pairs)), true};
      }
    }
    const int64_t units = tiles * num_kb;
    if (pair_mode != 2 && ws_bytes >= sk_bytes(sms, bn, tiles) && units >= 2 * (int64_t)sms && tiles % sms != 0) {
      const double share = (double)units / sms;
      const double contributors = 1.0 + (double)num_kb / share;
      const double sk = (share + (32.0 + 8.0 * contributors) * bn / 256.0) * per_kb;
      if (sk < best_cost || (force_sk && !best.stream_k)) {
        best_cost = force_sk ? 0.0 : sk;
        best = Plan{bn, true, (unsigned)sms};
      }
    }
  }
  best.cost = best_cost;
  return best;
}

template <bool A4, bool B4>
int launch_bn(const void* a, int64_t lda, const void* b, int64_t ldb, const GemmParams& p, const Plan& plan, cudaStream_t st) {
  if constexpr (!B4) {
    if (plan.pair) {
      switch (plan.bn) {
        case 256: return launch_gemm<256, A4, false, true>(a, lda, b, ldb, p, plan, st);
        case 192: return launch_gemm<192, A4, false, true>(a, lda, b, ldb, p, plan, st);
        case 64: return launch_gemm<64, A4, false, true>(a, lda, b, ldb, p, plan, st);
        default: return launch_gemm<128, A4, false, true>(a, lda, b, ldb, p, plan, st);
      }
    }
  }
  switch (plan.bn) {
    case 256: return launch_gemm<256, A4, B4>(a, lda, b, ldb, p, plan, st);
    case 192: return launch_gemm<192, A4, B4>(a, lda, b, ldb, p, plan, st);
    case 64: return launch_gemm<64, A4, B4>(a, lda, b, ldb, p, plan, st);
    default: return launch_gemm<128, A4, B4>(a, lda, b, ldb, p, plan, st);
  }
}

}  // namespace
}  // namespace hot

extern "C" size_t hot_gemm_i8_workspace_bytes(int64_t M, int64_t N) {
  const int sms = hot::device_sm_count();
  if (sms <= 0 || M <= 0 || N <= 0) return 0;
  size_t need = 0;
  for (int bn : {256, 192, 128, 64}) {
    const size_t b = hot::sk_bytes(sms, bn, hot::tiles_for((int)M, (int)N, bn));
    if (b > need) need = b;
  }
  return need;
}

extern "C" int hot_gemm_i8_ws(const void* a, int a_storage, int64_t lda, const void* b, int b_storage, int64_t ldb,
                              int64_t M, int64_t N, int64_t K, const float* scale_a, int scale_a_per_row,
                              const float* scale_b, int scale_b_per_row, float post, void* out, int out_dtype, int64_t ldo,
                              void* workspace, size_t workspace_bytes, uint32_t* status_word, hot_stream_t stream) {
  using namespace hot;
  if (!a || !b || !out) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8: null pointer");
  if (M <= 0 || N <= 0 || K <= 0 || M > (1 << 30) || N > (1 << 30) || K > (1 << 30))
    HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8: bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (out_dtype != HOT_I32 && (!scale_a || !scale_b)) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8: null scale pointer");
  const bool a4 = a_storage == HOT_STORE_INT4, b4 = b_storage == HOT_STORE_INT4;
  if ((a4 || b4) && (K % 2 != 0)) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8: packed INT4 operands need an even K");
  const int64_t abytes = a4 ? (K + 15) / 16 * 8 : K, bbytes = b4 ? (K + 15) / 16 * 8 : K;  // packed: whole runs of 16 codes
  if (lda % 16 || ldb % 16 || lda < abytes || ldb < bbytes || ((uintptr_t)a) % 16 || ((uintptr_t)b) % 16)
    HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8: operand base and pitch must be 16-byte aligned and cover K");
  if (ldo < N) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8: ldo < N");
  const int osz = out_dtype == HOT_BF16 ? 2 : 4;
  if (out_dtype != HOT_F32 && out_dtype != HOT_BF16 && out_dtype != HOT_I32)
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_gemm_i8: out dtype %d", out_dtype);
  if (((uintptr_t)out) % 16 != 0 || (ldo * osz) % 4 != 0) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8: out must be 16-byte aligned");
  GemmParams p;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.num_kb = (int)((K + kBK - 1) / kBK);
  p.sa = scale_a;
  p.sb = scale_b;
  if (scale_a_per_row < 0) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8: scale_a_per_row must be 0, 1 or a row count");
  p.sa_row = scale_a_per_row;
  p.sb_row = scale_b_per_row ? 1 : 0;
  p.group_kb = 0;
  p.ga = p.gb = nullptr;
  p.post = post;
  p.out = out;
  p.ldo = ldo;
  p.out_dtype = out_dtype;
  p.status = status_word;
  p.wait_ns = wait_limit_ns();
  cudaStream_t st = (cudaStream_t)stream;
  const int sms = device_sm_count();
  if (sms <= 0) return HOT_ERR_CUDA;
  if (workspace && ((uintptr_t)workspace) % 16 != 0) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_ws: workspace must be 16-byte aligned");
  const Plan plan = make_plan(p.M, p.N, p.num_kb, sms, workspace ? workspace_bytes : 0, !b4, a4 || b4);
  p.stream_k = plan.stream_k ? 1 : 0;
  p.sk_partials = nullptr;
  p.sk_counters = nullptr;
  if (plan.stream_k) {
    const int64_t tiles = tiles_for(p.M, p.N, plan.bn);
    p.sk_partials = (int32_t*)workspace;
    p.sk_counters = (uint32_t*)((uint8_t*)workspace + (size_t)2 * sms * kBM * plan.bn * sizeof(int32_t));
    HOT_CUDA(cudaMemsetAsync(p.sk_counters, 0, (size_t)tiles * sizeof(uint32_t), st));
  }
  if (!a4 && !b4) return launch_bn<false, false>(a, lda, b, ldb, p, plan, st);
  if (a4 && !b4) return launch_bn<true, false>(a, lda, b, ldb, p, plan, st);
  if (!a4 && b4) return launch_bn<false, true>(a, lda, b, ldb, p, plan, st);
  return launch_bn<true, true>(a, lda, b, ldb, p, plan, st);
}

extern "C" int hot_gemm_i8(const void* a, int a_storage, int64_t lda, const void* b, int b_storage, int64_t ldb,
                           int64_t M, int64_t N, int64_t K, const float* scale_a, int scale_a_per_row,
                           const float* scale_b, int scale_b_per_row, float post, void* out, int out_dtype, int64_t ldo,
                           uint32_t* status_word, hot_stream_t stream) {
  return hot_gemm_i8_ws(a, a_storage, lda, b, b_storage, ldb, M, N, K, scale_a, scale_a_per_row, scale_b, scale_b_per_row,
                        post, out, out_dtype, ldo, nullptr, 0, status_word, stream);
}

extern "C" int hot_gemm_i8_grouped(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t M, int64_t N,
                                   int64_t groups, int64_t group_k, const float* scale_a, int scale_a_per_row,
                                   const float* scale_b, float post, void* out, int out_dtype, int64_t ldo,
                                   uint32_t* status_word, hot_stream_t stream) {
  using namespace hot;
  if (!a || !b || !out || !scale_a || !scale_b) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_grouped: null pointer");
  if (M <= 0 || N <= 0 || groups <= 0 || group_k <= 0 || M > (1 << 30) || N > (1 << 30) || groups * group_k > (1 << 30))
    HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_grouped: bad shape M=%lld N=%lld groups=%lld group_k=%lld", (long long)M, (long long)N,
             (long long)groups, (long long)group_k);
  if (group_k % kBK != 0)
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_gemm_i8_grouped: group_k %lld must be a multiple of %d (pad each group with zero codes)",
             (long long)group_k, kBK);
  const int64_t K = groups * group_k;
  if (lda % 16 || ldb % 16 || lda < K || ldb < K || ((uintptr_t)a) % 16 || ((uintptr_t)b) % 16)
    HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_grouped: operand base and pitch must be 16-byte aligned and cover groups * group_k");
  if (out_dtype != HOT_F32 && out_dtype != HOT_BF16) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_gemm_i8_grouped: out dtype %d", out_dtype);
  const int osz = out_dtype == HOT_BF16 ? 2 : 4;
  if (ldo < N || ((uintptr_t)out) % 16 != 0 || (ldo * osz) % 16 != 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_grouped: out and its pitch must be 16-byte aligned, ldo >= N");
  GemmParams p;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.num_kb = (int)(K / kBK);
  p.sa = p.sb = nullptr;
  p.sa_row = scale_a_per_row ? 1 : 0;
  p.sb_row = 0;
  p.group_kb = (int)(group_k / kBK);
  p.ga = scale_a;
  p.gb = scale_b;
  p.post = post;
  p.out = out;
  p.ldo = ldo;
  p.out_dtype = out_dtype;
  p.status = status_word;
  p.wait_ns = wait_limit_ns();
  p.stream_k = 0;
  p.sk_partials = nullptr;
  p.sk_counters = nullptr;
  const int sms = device_sm_count();
  if (sms <= 0) return HOT_ERR_CUDA;
  const int64_t tiles = tiles_for(p.M, p.N, 128);
  const Plan plan{128, false, (unsigned)(tiles < sms ? tiles : sms)};
  return launch_gemm<128, false, false, false, true>(a, lda, b, ldb, p, plan, (cudaStream_t)stream);
}

namespace hot {
namespace {
// Validates one problem of hot_gemm_i8_dual and turns it into kernel parameters.
int fill_problem(const hot_gemm_problem_t* g, bool allow_packed_a, GemmParams* p, const char* who) {
  if (!g || !g->a || !g->b || !g->out) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_dual: %s: null pointer", who);
  if (g->M <= 0 || g->N <= 0 || g->K <= 0 || g->M > (1 << 30) || g->N > (1 << 30) || g->K > (1 << 30))
    HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_dual: %s: bad shape", who);
  const bool a4 = g->a_storage == HOT_STORE_INT4;
  if (a4 && !allow_packed_a) HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_gemm_i8_dual: %s: packed INT4 is taken for the main problem's A only", who);
  if (a4 && g->K % 2 != 0) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_dual: %s: packed INT4 operands need an even K", who);
  const int64_t abytes = a4 ? (g->K + 15) / 16 * 8 : g->K;
  if (g->lda % 16 || g->ldb % 16 || g->lda < abytes || g->ldb < g->K || ((uintptr_t)g->a) % 16 || ((uintptr_t)g->b) % 16)
    HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_dual: %s: operand base and pitch must be 16-byte aligned and cover K", who);
  if (g->out_dtype != HOT_F32 && g->out_dtype != HOT_BF16 && g->out_dtype != HOT_I32)
    HOT_FAIL(HOT_ERR_UNSUPPORTED, "hot_gemm_i8_dual: %s: out dtype %d", who, g->out_dtype);
  if (g->out_dtype != HOT_I32 && (!g->scale_a || !g->scale_b)) HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_dual: %s: null scale pointer", who);
  const int osz = g->out_dtype == HOT_BF16 ? 2 : 4;
  if (g->ldo < g->N || ((uintptr_t)g->out) % 16 != 0 || (g->ldo * osz) % 4 != 0 || g->scale_a_per_row < 0)
    HOT_FAIL(HOT_ERR_ARG, "hot_gemm_i8_dual: %s: bad output pitch / alignment / scale layout", who);
  *p = GemmParams{};
  p->M = (int)g->M;
  p->N = (int)g->N;
  p->K = (int)g->K;
  p->num_kb = (int)((g->K + kBK - 1) / kBK);
  p->sa = g->scale_a;
  p->sb = g->scale_b;
  p->sa_row = g->scale_a_per_row;
  p->sb_row = g->scale_b_per_row ? 1 : 0;
  p->post = g->post;
  p->out = g->out;
  p->ldo = g->ldo;
  p->out_dtype = g->out_dtype;
  return HOT_OK;
}

// k-blocks of the busiest worker under the dual schedule of SegmentIter (same rules, on the host); t1 rider
// pieces of kb1 k-blocks each
int64_t dual_max_load(int64_t t0, int kb0, int64_t t1, int kb1, int workers) {
  const int lag = (kb1 + kb0 / 2) / kb0;
  const int64_t free_w = workers - t1;
  int64_t worst = 0;
  for (int w = 0; w < workers; ++w) {
    int64_t load = w < t1 ? kb1 : 0;
    for (int round = 0;; ++round) {
      const bool all = round >= lag;
      const int64_t base = all ? lag * free_w + (round - lag) * (int64_t)workers : round * free_w;
      if (base >= t0) break;
      const int64_t rank = all ? w : w - t1;
      if (rank < 0) continue;
      if (base + rank >= t0) break;
      load += kb0;
    }
    if (load > worst) worst = load;
  }
  return worst;
}
}  // namespace
}  // namespace hot

namespace hot {
// hot_gemm_i8_dual with scratch: `workspace` (256-byte aligned) for the partial sums of rider tiles that are cut
// along K, `counters` = 160 zeroed words (left zero).  Without them rider tiles stay whole.
int gemm_i8_dual_ws(const hot_gemm_problem_t* main_problem, const hot_gemm_problem_t* rider_problem, void* workspace,
                    size_t workspace_bytes, uint32_t* counters, uint32_t* status_word, hot_stream_t stream) {
  GemmParams p0, p1;
  if (int rc = fill_problem(main_problem, true, &p0, "main problem")) return rc;
  if (int rc = fill_problem(rider_problem, false, &p1, "rider problem")) return rc;
  p0.status = p1.status = status_word;
  p0.wait_ns = p1.wait_ns = wait_limit_ns();
  cudaStream_t st = (cudaStream_t)stream;
  const int sms = device_sm_count();
  if (sms <= 0) return HOT_ERR_CUDA;
  const bool a4 = main_problem->a_storage == HOT_STORE_INT4;
  // One launch pays when the rider's few long tiles fit beside the main problem's last, partly empty
  // wave; otherwise (or with HOT_GEMM_DUAL=0) the two problems run one after the other.  The tile
  // width, and into how many stretches of k-blocks a rider tile is cut, are those whose busiest worker,
  // replayed on the host, has the least to do.
  const char* env = getenv("HOT_GEMM_DUAL");
  const char* senv = getenv("HOT_GEMM_RIDER_SPLIT");  // 1: rider tiles stay whole; n: cut into n where possible
  const int force_split = senv ? atoi(senv) : 0;
  // The decision depends on the shapes and the switches only; a training step asks for the same few again and
  // again, and the replay below costs tens of microseconds of host time, so the answers are kept.
  struct Decision {
    int key[13];
    Plan s0, s1;
    int dual_bn, dual_split;
    bool dual;
  };
  static std::mutex cache_mutex;
  static std::vector<Decision> cache;
  const char* e1 = getenv("HOT_GEMM_SCHEDULE");
  const char* e2 = getenv("HOT_GEMM_PAIR");
  const bool split_ok = workspace && counters && ((uintptr_t)workspace) % 16 == 0;
  const int key[13] = {p0.M, p0.N, p0.K, p1.M, p1.N, p1.K, sms, a4 ? 1 : 0, (env ? env[0] : 0) | ((e1 ? e1[0] : 0) << 8) | ((e2 ? e2[0] : 0) << 16),
                       force_split, split_ok ? 1 : 0, (int)(uint32_t)(workspace_bytes & 0xFFFFFFFFu), (int)(uint32_t)(workspace_bytes >> 32)};
  Decision dec;
  bool have = false;
  {
    std::lock_guard<std::mutex> lock(cache_mutex);
    for (const Decision& d : cache)
      if (memcmp(d.key, key, sizeof(key)) == 0) {
        dec = d;
        have = true;
        break;
      }
  }
  if (!have) {
  const Plan s0 = make_plan(p0.M, p0.N, p0.num_kb, sms, 0, !a4, a4), s1 = make_plan(p1.M, p1.N, p1.num_kb, sms, 0, true, false);
  int dual_bn = 0, dual_split = 1;
  double together = 0.0;
  for (int bn : {256, 192}) {
    const int64_t t0 = tiles_for(p0.M, p0.N, bn), t1 = tiles_for(p1.M, p1.N, bn);
    if (t1 > sms || t0 < sms || t1 < 1) continue;
    for (int split = 1; split <= 4; ++split) {
      if (force_split > 0 ? split != force_split : split > 2) continue;  // more than two stretches only when asked (tests)
      const int piece = (p1.num_kb + split - 1) / split;
      if (split > 1) {
        // every stretch non-empty, a slot per worker with a stretch, a counter per rider tile
        if (!workspace || !counters || t1 * split > sms || (int64_t)(split - 1) * piece >= p1.num_kb || t1 > 160 ||
            (size_t)(t1 * split) * kBM * bn * sizeof(int32_t) > workspace_bytes || ((uintptr_t)workspace) % 16 != 0)
          continue;
      }
      // Whoever completes a cut tile reads every stretch's sums back from L2, chunk by chunk, and adds them; with the
      // parking of the sums before it that costs the busiest worker about 10 us for two stretches and more for
      // three or four (measured on B200 at ViT-B sizes: 768 x 768 x 6304 beside 12608 x 768 x 768 gains 2 us from
      // a cut in two and loses with three or four; larger riders lose with two), some 14000 units of this model.
      const double fix = split > 1 ? 14000.0 + 4000.0 * (split - 2) : 0.0;
      const double c = (double)dual_max_load(t0, p0.num_kb, t1 * split, piece, sms) * (bn + 400.0) + fix;
      if (!dual_bn || c < together) {
        dual_bn = bn;
        dual_split = split;
        together = c;
      }
    }
  }
  bool dual = dual_bn != 0 && !(env && env[0] == '0');
  // a second launch costs about 3 us of ramp-down and ramp-up, some 4000 units of this model
  if (dual && !(env && env[0] == '1')) dual = together < s0.cost + s1.cost + 4000.0;
    memcpy(dec.key, key, sizeof(key));
    dec.s0 = s0;
    dec.s1 = s1;
    dec.dual_bn = dual_bn;
    dec.dual_split = dual_split;
    dec.dual = dual;
    std::lock_guard<std::mutex> lock(cache_mutex);
    if (cache.size() >= 256) cache.clear();
    cache.push_back(dec);
  }
  const Plan &s0 = dec.s0, &s1 = dec.s1;
  const int dual_bn = dec.dual_bn, dual_split = dec.dual_split;
  const bool dual = dec.dual;
  if (dual) {
    p1.split = dual_split;
    p1.sk_partials = (int32_t*)workspace;
    p1.sk_counters = counters;
    Rider r{rider_problem->a, rider_problem->lda, rider_problem->b, rider_problem->ldb, p1};
    const Plan plan{dual_bn, false, (unsigned)sms};
    const void* a = main_problem->a;
    const void* b = main_problem->b;
    const int64_t lda = main_problem->lda, ldb = main_problem->ldb;
    if (dual_bn == 256) {
      if (a4) return launch_gemm<256, true, false>(a, lda, b, ldb, p0, plan, st, &r);
      return launch_gemm<256, false, false>(a, lda, b, ldb, p0, plan, st, &r);
    }
    if (a4) return launch_gemm<192, true, false>(a, lda, b, ldb, p0, plan, st, &r);
    return launch_gemm<192, false, false>(a, lda, b, ldb, p0, plan, st, &r);
  }
  int rc = a4 ? launch_bn<true, false>(main_problem->a, main_problem->lda, main_problem->b, main_problem->ldb, p0, s0, st)
              : launch_bn<false, false>(main_problem->a, main_problem->lda, main_problem->b, main_problem->ldb, p0, s0, st);
  if (rc) return rc;
  return launch_bn<false, false>(rider_problem->a, rider_problem->lda, rider_problem->b, rider_problem->ldb, p1, s1, st);
}
}  // namespace hot

extern "C" int hot_gemm_i8_dual(const hot_gemm_problem_t* main_problem, const hot_gemm_problem_t* rider_problem,
                                uint32_t* status_word, hot_stream_t stream) {
  return hot::gemm_i8_dual_ws(main_problem, rider_problem, nullptr, 0, nullptr, status_word, stream);
}
