// Stage 2, Blackwell kernel: block-sparse attention forward with TMA + tcgen05 + TMEM.
//
// Replaces sparseattention/sparse_attn_kernel.py:72-146 (kernel) and 10-63 (inner loop)
// for fp16 / bf16, head dim 64 or 128, BLOCK_Q = 128 and BLOCK_K in {32, 64, 128}.
//
// Persistent grid: one CTA per SM (384 threads) works through (query block, batch, head) tiles drawn
// from a device-wide counter (tiles differ in length); the loads and first MMAs of a tile overlap the
// epilogue of the previous one (Q is double-buffered, barrier phases run on across tiles).  For a tile --
// one query block (128 rows) of one (batch, head) -- the CTA walks its two kv-block lists -- the full list first, then the partial list: the order of
// sparse_attn_kernel.py:113-142 -- in steps of 128 kv rows (128 / BLOCK_K listed blocks):
//
//   warp 0     K producer.  Reads the lists and gathers the listed kv blocks of K into 128-row,
//              128-byte-swizzled tiles of a two-stage shared-memory ring with TMA tile loads whose
//              row coordinate comes from the list (eight lanes issue the eight boxes of a tile),
//              plus the 512-byte bit-mask tiles of the partial blocks (cp.async.bulk from the
//              packed plane of stage 1, four-stage ring).
//   warp 1     V producer: the same for V, two-stage ring.
//   warp 2     S issuer.  S(j) = Q.K(j)^T into one of two score buffers in tensor memory
//              (tcgen05.mma, both operands in shared memory), one step ahead of the softmax.
//   warp 3     P.V issuer.  O += P(j).V(j) with P read from its own buffer in tensor memory.
//   warps 4-11 softmax; a thread owns a query row and one half of the 128 score columns.  Scores
//              are exponentiated against the row's running reference max in a single pass (base 2,
//              scale folded as in sparse_attn_kernel.py:152; a row's first scores are tried against
//              0); the reference moves, and O is rescaled in tensor memory, only when a score
//              exceeds it by more than 2^8 (the pass is then redone from the intact scores).  Steps that contain a partial or padding block apply
//              the bit mask; steps of full blocks do no mask work.  P is rounded to the V dtype
//              (line 61); row sums stay in fp32 (line 57).  Finally O / l is staged in the tile's Q
//              slot and written with one TMA store per warp; a row with no attended key yields 0
//              (the reference yields NaN, line 53).
//
// Tensor memory (512 columns): score buffers at 0 and 128, O at 256, P buffers at 384 and 448.
//
// A step whose last slots run past the end of the lists re-loads the first listed block with an
// all-zero mask word.  Every mbarrier wait is bounded; on expiry the CTA reports
// SA_DEV_WAIT_EXPIRED, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "ptx_sm100.cuh"
#include "sa_common.cuh"

namespace sa {
namespace {

constexpr int kTileM = 128;          // query rows per CTA (= BLOCK_Q)
constexpr int kTileN = 128;          // kv rows per MMA step
constexpr int kSplit = 2;            // threads per query row in the softmax (column groups)
constexpr int kThreadsTC = 128 + 128 * kSplit;   // warps: K producer, V producer, S issuer, P.V issuer, 4 * kSplit softmax
constexpr int kSoftmaxWarp0 = 4;     // first softmax warp (a multiple of 4: TMEM lane quarter = warp % 4)
constexpr uint32_t kTmemCols = 512;  // score buffers at columns 0 and 128, O at 256, P buffers at 384 and 448
constexpr int kStagesK = 2;          // K tiles in flight in shared memory
constexpr int kStagesV = 2;          // V tiles in flight in shared memory
constexpr int kBitStages = 4;        // steps of bit-mask tiles in flight
constexpr int kTileRing = 4;         // tile indices the scheduling warp may be ahead of the slowest role
constexpr uint32_t kPanelBytes = 128u * 128u;   // 128 rows x 64 elements x 2 B
constexpr float kRescaleThreshold = 8.0f;       // log2 units
constexpr float kFreshFloor = -4.0f;            // a row's first scores are taken against 0 if their max is in [-4, 8]
enum Bar : int {
  BAR_Q_FULL = 0,                                  // 2: Q tile of a query block landed
  BAR_Q_EMPTY = BAR_Q_FULL + 2,                    // 2: last S of the tile that used the Q slot complete
  BAR_K_FULL = BAR_Q_EMPTY + 2,                                      // kStagesK: K tile landed
  BAR_K_EMPTY = BAR_K_FULL + kStagesK,             // kStagesK: K tile consumed by S = Q.K^T
  BAR_V_FULL = BAR_K_EMPTY + kStagesK,             // kStagesV
  BAR_V_EMPTY = BAR_V_FULL + kStagesV,             // kStagesV: V tile consumed by O += P.V
  BAR_S_FULL = BAR_V_EMPTY + kStagesV,             // 2: scores of buffer j & 1 complete
  BAR_P_FULL = BAR_S_FULL + 2,                     // 2: P of buffer j & 1 written (and S read) by all softmax threads
  BAR_PV_DONE = BAR_P_FULL + 2,                    // 2: O += P.V of step j complete (barrier j & 1)
  BAR_O_FULL = BAR_PV_DONE + 2,                    // last O += P.V of a tile complete
  BAR_O_FREE,                                      // the epilogue has read O out of tensor memory
  BAR_BITS_EMPTY,                                  // kBitStages: bit-mask tiles of a masked step read by the softmax
  BAR_Q_STORED = BAR_BITS_EMPTY + kBitStages,      // 2: the O tile staged in the Q slot has been read by its store
  BAR_TILE_FULL = BAR_Q_STORED + 2,                // kTileRing: a tile index has been published
  BAR_TILE_EMPTY = BAR_TILE_FULL + kTileRing,      // kTileRing: every other role has read it
  BAR_COUNT = BAR_TILE_EMPTY + kTileRing
};

template <int D>
struct Smem {
  static constexpr uint32_t kTileBytes = kPanelBytes * (D / 64);
  static constexpr uint32_t off_q = 0;
  static constexpr uint32_t off_k = 2 * kTileBytes;              // two Q tiles first
  static constexpr uint32_t off_v = off_k + kStagesK * kTileBytes;
  static constexpr uint32_t off_bits = off_v + kStagesV * kTileBytes;      // [kBitStages][4 sub-slots][128 rows] u32
  static constexpr uint32_t off_bar = off_bits + kBitStages * 4 * 128 * 4;
  static constexpr uint32_t off_misc = off_bar + 8 * 48;
  static constexpr uint32_t off_ids = off_misc + 16 + 16 * kTileRing;  // misc: TMEM base, abort flag, tile ring (index and the two list lengths per slot)
  static constexpr uint32_t off_xch = off_ids + 2 * 4 * 4 * 4;         // ids: per producer warp [4 steps][4 entries]; xch: [2 parities + epilogue][kSplit column groups][128 rows] f32
  static constexpr uint32_t total = off_xch + 3 * kSplit * 128 * 4;
  static constexpr uint32_t dynamic_bytes = total + 1024;       // slack to align the base to 1024 B
};
static_assert(BAR_COUNT <= 48, "barrier area too small");

template <typename T> struct Fmt;
template <> struct Fmt<__half> {
  static constexpr uint32_t umma = 0;
  static __device__ __forceinline__ uint32_t pack2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <> struct Fmt<__nv_bfloat16> {
  static constexpr uint32_t umma = 1;
  static __device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// 32 score columns of one thread: x = s*scale - m_ref, masked columns -> -inf (kMasked), P = exp2(x)
// rounded to T into pk, fp32 sum of the unrounded P (lines 54, 57, 61) and max of x.
// The running max and sum are kept in kAcc independent accumulators each (pair i goes to i % kAcc), so
// that consecutive pairs do not wait for one another's result.
constexpr int kAcc = 2;
template <typename T, bool kMasked>
__device__ __forceinline__ void softmax_chunk(const uint32_t (&r)[32], uint32_t w, uint64_t scale2, uint64_t nm2,
                                              uint32_t (&pk)[16], uint64_t (&sum2v)[kAcc], float (&xmaxv)[kAcc]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    uint64_t& sum2 = sum2v[i % kAcc];
    float& xmax = xmaxv[i % kAcc];
    float x0, x1;
    ptx::unpack_f32x2(ptx::fma_f32x2(ptx::pack_u32x2(r[2 * i], r[2 * i + 1]), scale2, nm2), x0, x1);
    if (kMasked) {
      x0 = (w >> (2 * i)) & 1u ? x0 : -INFINITY;                 // line 47
      x1 = (w >> (2 * i + 1)) & 1u ? x1 : -INFINITY;
    }
    xmax = ptx::max3(xmax, x0, x1);
    const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
    sum2 = ptx::add_f32x2(sum2, ptx::pack_f32x2(p0, p1));
    pk[i] = Fmt<T>::pack2(p0, p1);
  }
}

// One pass over this thread's kCW score columns, kCW / 32 chunks of 32.  w[c] is the bit-mask word
// of chunk c for this thread's row; a warp covers 32 rows, so on masked steps a chunk is one 32 x 32
// block of the mask.  A block that is False for all 32 rows costs no arithmetic (P = 0, no
// exponentials); one that is True for all 32 rows takes the mask-free arithmetic.
template <typename T, bool kMasked, int kCW>
__device__ __forceinline__ void softmax_pass(uint32_t t_s, uint32_t t_p, float scale, float m_ref,
                                             const uint32_t (&w)[kCW / 32], float& sum_out, float& xmax_out) {
  constexpr int kChunks = kCW / 32;
  bool dead[kChunks], solid[kChunks];
  uint32_t r[kChunks][32];
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    dead[c] = kMasked && __all_sync(0xffffffffu, w[c] == 0u);
    solid[c] = !kMasked || __all_sync(0xffffffffu, w[c] == 0xffffffffu);
    ptx::tmem_ld32(t_s + 32 * c, r[c]);
  }
  ptx::tmem_ld_wait();
  const uint64_t scale2 = ptx::pack_f32x2(scale, scale);
  const uint64_t nm2 = ptx::pack_f32x2(-m_ref, -m_ref);
  uint64_t sum2[kAcc];
  float xmax[kAcc];
#pragma unroll
  for (int a = 0; a < kAcc; ++a) { sum2[a] = ptx::pack_f32x2(0.f, 0.f); xmax[a] = -INFINITY; }
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    uint32_t pk[16];
    if (dead[c]) {
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[i] = 0u;
    } else if (solid[c]) {
      softmax_chunk<T, false>(r[c], w[c], scale2, nm2, pk, sum2, xmax);
    } else {
      softmax_chunk<T, true>(r[c], w[c], scale2, nm2, pk, sum2, xmax);
    }
    ptx::tmem_st16(t_p + 16 * c, pk);
  }
#pragma unroll
  for (int a = 1; a < kAcc; ++a) { sum2[0] = ptx::add_f32x2(sum2[0], sum2[a]); xmax[0] = fmaxf(xmax[0], xmax[a]); }
  float s0, s1;
  ptx::unpack_f32x2(sum2[0], s0, s1);
  sum_out = s0 + s1;
  xmax_out = xmax[0];
}

// Moves kCols fp32 columns between tensor memory and registers (kCols = 32 or 16).
template <int kCols>
__device__ __forceinline__ void tmem_load_cols(uint32_t taddr, uint32_t (&r)[kCols]) {
  if constexpr (kCols == 32) ptx::tmem_ld32(taddr, r); else ptx::tmem_ld16(taddr, r);
}
template <int kCols>
__device__ __forceinline__ void tmem_store_cols(uint32_t taddr, const uint32_t (&r)[kCols]) {
  if constexpr (kCols == 32) ptx::tmem_st32(taddr, r); else ptx::tmem_st16(taddr, r);
}

// The rare second pass of a step, after the reference max of some row moved, out of line so that the
// hot loop stays small: rescales this thread's O columns by alpha (sparse_attn_kernel.py:58) when
// asked to, then redoes the pass from the intact scores against m_ref.  Returns the new row sum.
template <typename T, int kCW, int kOC>
__device__ __noinline__ float second_pass_cold(uint32_t t_s, uint32_t t_p, uint32_t t_o, float scale, float m_ref,
                                               float alpha, bool rescale_o, uint32_t pv_bar, uint32_t pv_parity,
                                               volatile int* abort_flag, uint32_t w0, uint32_t w1) {
  constexpr int kOChunk = kOC > 32 ? 32 : kOC;
  if (rescale_o) {
    // O must hold every product up to the previous step before it is rescaled.
    ptx::mbar_wait(pv_bar, pv_parity, abort_flag);
    ptx::tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < kOC / kOChunk; ++c) {
      uint32_t r[kOChunk];
      tmem_load_cols<kOChunk>(t_o + c * kOChunk, r);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < kOChunk; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
      tmem_store_cols<kOChunk>(t_o + c * kOChunk, r);
    }
  }
  static_assert(kCW / 32 <= 2, "the out-of-line pass takes two mask words");
  uint32_t w[kCW / 32];
  w[0] = w0;
  if (kCW / 32 > 1) w[kCW / 32 - 1] = w1;
  float sum, xmax;
  softmax_pass<T, true, kCW>(t_s, t_p, scale, m_ref, w, sum, xmax);
  return sum;
}

// Work of one tile -- a (query block, batch, head) or, when the walks are split, one of p.splits
// contiguous ranges of its steps -- read from the lists.
struct TileInfo {
  int b, h, qblk;
  int b_out;                  // batch index of the output: the split's own slab of the partial results
  int n_full, n_part, total;
  int j0, j1, n_steps;        // steps [j0, j1) of the walk over the two lists; n_steps = j1 - j0
  int n_plain;                // leading steps of the whole walk made of full blocks only
  int m0;                     // first step of the range that carries mask words (may be >= j1)
};

// The two list lengths of a tile's (query block, batch, head), read from global memory: by the
// scheduling warp only, which hands them to the other roles with the tile index.
__device__ __forceinline__ void tile_lens(const AttnParams& p, int tile, int nq, int& n_full, int& n_part) {
  const int unit = tile / p.splits;
  const int bh = unit / nq, qblk = unit % nq;
  const int b = bh / p.H, h = bh % p.H;
  n_full = p.full_lens[b * p.fls[0] + h * p.fls[1] + static_cast<int64_t>(qblk) * p.fls[2]];  // line 107
  n_part = p.part_lens[b * p.pls[0] + h * p.pls[1] + static_cast<int64_t>(qblk) * p.pls[2]];  // line 127
}

// Out of line: every role calls it once per tile, and one copy keeps the kernel's code small.
__device__ __noinline__ TileInfo tile_info(const AttnParams& p, int tile, int n_full, int n_part, int nq, int nk,
                                           int eps_shift) {
  TileInfo t;
  // (unsigned 32-bit divisions, and none where the divisor is 1: every role pays for this at each tile)
  const unsigned utile = static_cast<unsigned>(tile), usplits = static_cast<unsigned>(p.splits);
  const unsigned unit = usplits == 1u ? utile : utile / usplits;      // the splits of a unit are neighbours
  const unsigned split = usplits == 1u ? 0u : utile - unit * usplits;
  const unsigned bh = unit / static_cast<unsigned>(nq);
  t.qblk = static_cast<int>(unit - bh * static_cast<unsigned>(nq));
  t.b = static_cast<int>(bh / static_cast<unsigned>(p.H));
  t.h = static_cast<int>(bh - static_cast<unsigned>(t.b) * static_cast<unsigned>(p.H));
  t.n_full = min(max(n_full, 0), nk);
  t.n_part = min(max(n_part, 0), nk);
  t.total = t.n_full + t.n_part;
  const int all_steps = (t.total + (1 << eps_shift) - 1) >> eps_shift;
  // all_steps < 2^23 (two lists of Sk / 32 entries at most) and splits <= 256: the products fit 32 bits
  t.j0 = usplits == 1u ? 0 : static_cast<int>(static_cast<unsigned>(all_steps) * split / usplits);
  t.j1 = usplits == 1u ? all_steps : static_cast<int>(static_cast<unsigned>(all_steps) * (split + 1u) / usplits);
  t.n_steps = t.j1 - t.j0;
  t.n_plain = t.n_full >> eps_shift;
  t.m0 = max(t.n_plain, t.j0);
  t.b_out = static_cast<int>(split) * p.B + t.b;
  return t;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreadsTC, 1)
attn_fwd_tc_kernel(const __grid_constant__ AttnParams p,
                   const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_o,
                   const int n_tiles) {
  using L = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = ptx::smem_u32(smem);
  const uint32_t sQ = sbase + L::off_q, sK = sbase + L::off_k, sV = sbase + L::off_v;
  const uint32_t sBits = sbase + L::off_bits;
  const uint32_t* bits_smem = reinterpret_cast<const uint32_t*>(smem + L::off_bits);
  auto bar = [&](int i) { return sbase + L::off_bar + 8u * static_cast<uint32_t>(i); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_misc + 4);
  volatile int* tile_ring = reinterpret_cast<volatile int*>(smem + L::off_misc + 16);
  float* xch = reinterpret_cast<float*>(smem + L::off_xch);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The epilogue stages a tile of O in the Q slot it has finished with and stores it with TMA when a
  // thread's share of a row is one 128-byte swizzle row; otherwise the threads store their rows directly.
  constexpr bool kStageO = (D / kSplit) * sizeof(T) == 128;
  const int nq = p.Sq / kTileM;
  const int nk = p.Sk / p.BK;
  // BLOCK_K is 32, 64 or 128: list entries per step (4, 2, 1) and 32-column sub-slots per entry
  // (1, 2, 4) are powers of two, so the per-step index arithmetic is shifts.
  const int eps_shift = p.BK == 32 ? 2 : (p.BK == 64 ? 1 : 0);
  const int sps_shift = 2 - eps_shift;
  const int eps = 1 << eps_shift;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(bar(BAR_Q_FULL + i), 1);
      ptx::mbar_init(bar(BAR_Q_EMPTY + i), 1);
      ptx::mbar_init(bar(BAR_S_FULL + i), 1);
      ptx::mbar_init(bar(BAR_P_FULL + i), 4 * kSplit);      // one arrival per softmax warp
      ptx::mbar_init(bar(BAR_PV_DONE + i), 1);
      ptx::mbar_init(bar(BAR_Q_STORED + i), 4 * kSplit);
    }
    for (int i = 0; i < kStagesK; ++i) {
      ptx::mbar_init(bar(BAR_K_FULL + i), 1);
      ptx::mbar_init(bar(BAR_K_EMPTY + i), 1);
    }
    for (int i = 0; i < kStagesV; ++i) {
      ptx::mbar_init(bar(BAR_V_FULL + i), 1);
      ptx::mbar_init(bar(BAR_V_EMPTY + i), 1);
    }
    ptx::mbar_init(bar(BAR_O_FULL), 1);
    ptx::mbar_init(bar(BAR_O_FREE), 4 * kSplit);
    for (int i = 0; i < kBitStages; ++i) {
      ptx::mbar_init(bar(BAR_BITS_EMPTY + i), 4 * kSplit);
    }
    for (int i = 0; i < kTileRing; ++i) {
      ptx::mbar_init(bar(BAR_TILE_FULL + i), 1);
      ptx::mbar_init(bar(BAR_TILE_EMPTY + i), 3 + 4 * kSplit);    // V producer, two issuers, softmax warps
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tO = tmem_base + 256;   // score buffer s lives at tmem_base + 128 * s, P buffer s at 384 + 64 * s

  // Every role walks the same sequence of tiles and keeps the same running counts -- steps done (g),
  // masked steps done (gu), non-empty tiles done (tq) -- from which buffer indices and barrier
  // phases follow; nothing is reset between tiles, so the loads and the first MMAs of a tile overlap
  // the epilogue of the previous one.  The sequence starts at blockIdx.x; warp 0 draws each further
  // tile from a device-wide counter (or, without one, steps by gridDim.x) and publishes it to the
  // other roles through a small ring in shared memory; an index >= n_tiles ends every role's loop.
  // Ordinal `ord` of the sequence lives in ring slot ord % kTileRing.
  // A wait that fails (it ran out, or another thread's did) ends the role's loop; a warp takes that
  // decision as a whole, so that no lane is left alone in a warp-wide tensor-memory instruction.
  // Whole warps wait, also where one lane acts on the result: a lone lane polling a barrier (the other
  // lanes parked at the reconvergence point) notices its completion several times later than a full warp.
  auto next_tile_warp = [&](int ord, int& n_full, int& n_part) -> int {
    const int slot = ord % kTileRing;
    if (!__all_sync(0xffffffffu, ptx::mbar_wait(bar(BAR_TILE_FULL + slot), (ord / kTileRing) & 1, abort_flag))) return n_tiles;
    const int t = tile_ring[4 * slot];
    n_full = tile_ring[4 * slot + 1];
    n_part = tile_ring[4 * slot + 2];
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(bar(BAR_TILE_EMPTY + slot));
    return t;
  };
  if (warp < 2) {
    // ------------------------------------------------------------------ producers
    // Warp 0 gathers Q, the K tiles and the bit-mask tiles, warp 1 the V tiles.  The whole warp
    // runs the loop and waits for a free stage: lane 0 arms its barrier, lanes 0-7 each issue one
    // TMA box, lanes 0-3 fetch the list entries of a step.
    const bool is_k = warp == 0;
    const CUtensorMap* tm = is_k ? &tm_k : &tm_v;
    if (lane == 0) {
      ptx::prefetch_tensormap(tm);
      if (is_k) ptx::prefetch_tensormap(&tm_q);
    }
    const int n_stages = is_k ? kStagesK : kStagesV;
    const uint32_t s_tiles = is_k ? sK : sV;
    const int bar_full = is_k ? BAR_K_FULL : BAR_V_FULL, bar_empty = is_k ? BAR_K_EMPTY : BAR_V_EMPTY;
    const uint32_t slot_bytes = static_cast<uint32_t>(p.BK) * 128u;
    constexpr int kPanels = D / 64;
    const int c_of_lane = lane / kPanels, pnl_of_lane = lane % kPanels;
    const bool has_box = c_of_lane < eps;
    bool bad_index = false;
    bool ok = true;
    int st = 0, round = 0, gu = 0, tq = 0;
    const uint32_t s_ids = sbase + L::off_ids + static_cast<uint32_t>(warp) * 64u;
    const volatile int* ids_ring = reinterpret_cast<const volatile int*>(smem + L::off_ids + warp * 64);
    // lane 0 of warp 0 publishes tile `t`, with its two list lengths, as ordinal `ord` of the sequence
    auto publish = [&](int ord, int t, int n_full, int n_part) {
      const int slot = ord % kTileRing;
      if (ord >= kTileRing) ok = ptx::mbar_wait(bar(BAR_TILE_EMPTY + slot), (ord / kTileRing - 1) & 1, abort_flag);
      tile_ring[4 * slot] = (ok && *abort_flag == 0) ? t : n_tiles;    // after a failed wait every role is sent home
      tile_ring[4 * slot + 1] = n_full;
      tile_ring[4 * slot + 2] = n_part;
      ptx::mbar_arrive(bar(BAR_TILE_FULL + slot));
    };
    int ord = 0;
    int tile = blockIdx.x, len_f = 0, len_p = 0;
    if (is_k) {
      if (lane == 0) {
        if (tile < n_tiles) tile_lens(p, tile, nq, len_f, len_p);
        publish(0, tile, len_f, len_p);
      }
      len_f = __shfl_sync(0xffffffffu, len_f, 0);
      len_p = __shfl_sync(0xffffffffu, len_p, 0);
    } else {
      tile = next_tile_warp(0, len_f, len_p);
    }
    while (tile < n_tiles && ok) {
      // The next tile is drawn now and published after this one's loads are issued: the answer of
      // the atomic is not waited for until then.
      int drawn = 0;
      if (is_k && lane == 0)
        drawn = p.tile_counter != nullptr ? atomicAdd(p.tile_counter, 1) + static_cast<int>(gridDim.x)
                                          : tile + static_cast<int>(gridDim.x);
      const TileInfo ti = tile_info(p, tile, len_f, len_p, nq, nk, eps_shift);
      const int b = ti.b, h = ti.h, qblk = ti.qblk, n_full = ti.n_full, total = ti.total, n_steps = ti.n_steps,
                n_plain = ti.n_plain, j0 = ti.j0, j1 = ti.j1;
      if (n_steps != 0) {
      if (is_k) {                                   // Q tile of this query block, double-buffered
        const int qs = tq & 1;
        if (tq >= 2) {
          ok = ptx::mbar_wait(bar(BAR_Q_EMPTY + qs), ((tq >> 1) - 1) & 1, abort_flag);
          if (ok && kStageO) ok = ptx::mbar_wait(bar(BAR_Q_STORED + qs), ((tq >> 1) - 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
        }
        if (lane == 0) {
          if (ok) {
            const int qb = p.qs[0] ? b : 0, qh = p.qs[1] ? h : 0;
            ptx::mbar_arrive_expect_tx(bar(BAR_Q_FULL + qs), L::kTileBytes);
#pragma unroll
            for (int pnl = 0; pnl < D / 64; ++pnl)
              ptx::tma_load_4d(sQ + qs * L::kTileBytes + pnl * kPanelBytes, &tm_q, bar(BAR_Q_FULL + qs),
                               pnl * 64, qblk * kTileM, qh, qb);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
      }
      const int cb = is_k ? (p.ks[0] ? b : 0) : (p.vs[0] ? b : 0);
      const int ch = is_k ? (p.ks[1] ? h : 0) : (p.vs[1] ? h : 0);
      const int32_t* fids = p.full_ids + b * p.fis[0] + h * p.fis[1] + static_cast<int64_t>(qblk) * p.fis[2];
      const int32_t* pids = p.part_ids + b * p.pis[0] + h * p.pis[1] + static_cast<int64_t>(qblk) * p.pis[2];
      const uint32_t* bits_plane = p.bits + b * p.bits_sb + h * p.bits_sh;
      // The list entries of a step are copied to a four-step ring in shared memory two steps before
      // they are needed, asynchronously (one group per step): nothing waits for the lists' latency.
      auto fetch_ids = [&](int j) {
        if (lane < eps && j < j1) {
          const int e = (j << eps_shift) + lane;
          const int ee = e < total ? e : 0;         // slots past the end re-load the first listed block
          const int32_t* src = ee < n_full ? fids + ee * p.fis[3] : pids + (ee - n_full) * p.pis[3];   // line 33
          ptx::cp_async_4(s_ids + static_cast<uint32_t>((j & 3) * 4 + lane) * 4u, src);
        }
        ptx::cp_async_commit();
      };
      __syncwarp();                                     // every lane has read the previous tile's last entries
      fetch_ids(j0);
      fetch_ids(j0 + 1);
      for (int j = j0; j < j1 && ok; ++j) {
        fetch_ids(j + 2);
        ptx::cp_async_wait<2>();                        // the group of step j has landed
        __syncwarp();
        const uint32_t dst = s_tiles + st * L::kTileBytes;
        const uint32_t full_bar = bar(bar_full + st);
        // The bit-mask tiles of the partial blocks of step j land on the K tile's barrier: once
        // S(j) is complete the softmax finds them in shared memory without a wait of its own.
        const bool with_bits = is_k && j >= n_plain;
        const int u = gu + (j - ti.m0), bst = u % kBitStages;
        uint32_t tx_bytes = L::kTileBytes;
        if (with_bits) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int e = (j << eps_shift) + (c >> sps_shift);
            tx_bytes += (e >= n_full && e < total) ? 512u : 0u;
          }
        }
        if (round > 0) ok = ptx::mbar_wait(bar(bar_empty + st), (round - 1) & 1, abort_flag);
        if (ok && with_bits && u >= kBitStages)
          ok = ptx::mbar_wait(bar(BAR_BITS_EMPTY + bst), (u / kBitStages - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (ok && lane == 0) ptx::mbar_arrive_expect_tx(full_bar, tx_bytes);
        __syncwarp();
        int id_c = ids_ring[(j & 3) * 4 + (c_of_lane & 3)];
        if (static_cast<unsigned>(id_c) >= static_cast<unsigned>(nk)) { bad_index = bad_index || has_box; id_c = 0; }
        if (ok && has_box)
          ptx::tma_load_4d(dst + pnl_of_lane * kPanelBytes + c_of_lane * slot_bytes, tm, full_bar,
                           pnl_of_lane * 64, id_c * p.BK, ch, cb);
        if (with_bits) {
          const int c = lane & 3, ec = c >> sps_shift;
          int id_b = ids_ring[(j & 3) * 4 + ec];
          if (static_cast<unsigned>(id_b) >= static_cast<unsigned>(nk)) id_b = 0;
          const int e = (j << eps_shift) + ec;
          if (ok && lane < 4 && e >= n_full && e < total) {
            const int64_t kb32 = (static_cast<int64_t>(id_b) << sps_shift) + (c & ((1 << sps_shift) - 1));
            const uint32_t* src = bits_plane + kb32 * p.Sq + qblk * kTileM;
            ptx::bulk_load(sBits + static_cast<uint32_t>(bst * 4 + c) * 512u, src, 512u, full_bar);
          }
        }
        if (++st == n_stages) { st = 0; ++round; }
      }
      gu += max(j1 - ti.m0, 0);
      ++tq;
      }
      ++ord;
      if (is_k) {
        if (lane == 0) {
          if (drawn < 0 || drawn > n_tiles) drawn = n_tiles;
          len_f = len_p = 0;
          if (drawn < n_tiles) tile_lens(p, drawn, nq, len_f, len_p);   // this tile's loads are all under way by now
          publish(ord, drawn, len_f, len_p);
        }
        tile = __shfl_sync(0xffffffffu, drawn, 0);
        len_f = __shfl_sync(0xffffffffu, len_f, 0);
        len_p = __shfl_sync(0xffffffffu, len_p, 0);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      } else {
        tile = next_tile_warp(ord, len_f, len_p);
      }
    }
    if (is_k && __any_sync(0xffffffffu, bad_index) && lane == 0 && p.dev_status != nullptr)
      atomicMax(p.dev_status, SA_DEV_BAD_INDEX);
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------------ S issuer: S(g) = Q.K(g)^T  (line 40)
    // The whole warp walks the loop and waits (a lone lane polling a barrier notices its completion
    // several times later than a full warp does); lane 0 issues.
    {
      constexpr uint32_t idesc_s = ptx::umma_idesc_f16(Fmt<T>::umma, kTileM, kTileN, 0);
      const uint64_t dq = ptx::umma_desc_sw128(sQ, 16u);
      const uint32_t dq_lo0 = static_cast<uint32_t>(dq), d_hi = static_cast<uint32_t>(dq >> 32);
      const uint32_t dk_lo0 = static_cast<uint32_t>(ptx::umma_desc_sw128(sK, 16u));
      bool ok = true;
      int st = 0, round = 0, g = 0, tq = 0;
      for (int ord = 0; ok; ++ord) {
        int len_f, len_p;
        const int tile = next_tile_warp(ord, len_f, len_p);
        if (tile >= n_tiles) break;
        const TileInfo ti = tile_info(p, tile, len_f, len_p, nq, nk, eps_shift);
        if (ti.n_steps == 0) continue;
        const int qs = tq & 1;
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(bar(BAR_Q_FULL + qs), (tq >> 1) & 1, abort_flag));
        const uint32_t dq_lo = dq_lo0 + qs * (L::kTileBytes >> 4);
        for (int j = 0; j < ti.n_steps && ok; ++j, ++g) {
          // Score buffer g & 1 is reused: the softmax of step g-2 has read it once P(g-2) is complete.
          // (The P buffer of the same parity is still being read by O += P.V(g-2); the softmax of
          // step g waits for that product itself before it writes P.)
          if (g >= 2) ok = ptx::mbar_wait(bar(BAR_P_FULL + (g & 1)), ((g - 2) >> 1) & 1, abort_flag);
          if (ok) ok = ptx::mbar_wait(bar(BAR_K_FULL + st), round & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
          if (lane == 0) {
            const uint32_t tS = tmem_base + 128u * (g & 1);
            const uint32_t dk_lo = dk_lo0 + st * (L::kTileBytes >> 4);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              constexpr uint32_t kPanelStep = kPanelBytes >> 4;
              const uint32_t off = (kk / 4) * kPanelStep + (kk % 4) * 2u;      // (panel, 32-byte K slice) >> 4
              if (kk == 0) ptx::mma_ss_lo<false>(tS, dq_lo + off, dk_lo + off, d_hi, idesc_s);
              else         ptx::mma_ss_lo<true>(tS, dq_lo + off, dk_lo + off, d_hi, idesc_s);
            }
            ptx::mma_commit(bar(BAR_K_EMPTY + st));
            ptx::mma_commit(bar(BAR_S_FULL + (g & 1)));
            if (j == ti.n_steps - 1) ptx::mma_commit(bar(BAR_Q_EMPTY + qs));   // Q tile no longer needed
          }
          __syncwarp();
          if (++st == kStagesK) { st = 0; ++round; }
        }
        ++tq;
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ P.V issuer: O += P(g).V(g)  (line 61)
    {
      constexpr uint32_t idesc_o = ptx::umma_idesc_f16(Fmt<T>::umma, kTileM, D, 1);
      const uint64_t dv = ptx::umma_desc_sw128(sV, kPanelBytes);
      const uint32_t dv_lo0 = static_cast<uint32_t>(dv), dv_hi = static_cast<uint32_t>(dv >> 32);
      bool ok = true;
      int g = 0, tq = 0;
      for (int ord = 0; ok; ++ord) {
        int len_f, len_p;
        const int tile = next_tile_warp(ord, len_f, len_p);
        if (tile >= n_tiles) break;
        const TileInfo ti = tile_info(p, tile, len_f, len_p, nq, nk, eps_shift);
        if (ti.n_steps == 0) continue;
        for (int j = 0; j < ti.n_steps && ok; ++j, ++g) {
          ok = ptx::mbar_wait(bar(BAR_P_FULL + (g & 1)), (g >> 1) & 1, abort_flag);
          if (ok) ok = ptx::mbar_wait(bar(BAR_V_FULL + (g & 1)), (g >> 1) & 1, abort_flag);
          // the first product of a tile overwrites O: the previous tile's epilogue must have read it
          if (ok && j == 0 && tq >= 1) ok = ptx::mbar_wait(bar(BAR_O_FREE), (tq - 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
          if (lane == 0) {
            const uint32_t tP = tmem_base + 384u + 64u * (g & 1);
            const uint32_t dv_lo = dv_lo0 + (g & 1) * (L::kTileBytes >> 4);
            if (j == 0) {
#pragma unroll
              for (int kk = 0; kk < kTileN / 16; ++kk) {
                if (kk == 0) ptx::mma_ts_lo<false>(tO, tP + kk * 8u, dv_lo + kk * 128u, dv_hi, idesc_o);
                else         ptx::mma_ts_lo<true>(tO, tP + kk * 8u, dv_lo + kk * 128u, dv_hi, idesc_o);
              }
            } else {
#pragma unroll
              for (int kk = 0; kk < kTileN / 16; ++kk) {
                ptx::mma_ts_lo<true>(tO, tP + kk * 8u, dv_lo + kk * 128u, dv_hi, idesc_o);
              }
            }
            ptx::mma_commit(bar(BAR_V_EMPTY + (g & 1)));
            ptx::mma_commit(bar(BAR_PV_DONE + (g & 1)));
            if (j == ti.n_steps - 1) ptx::mma_commit(bar(BAR_O_FULL));
          }
          __syncwarp();
        }
        ++tq;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax
    // Thread = (query row, one of kSplit groups of 128 / kSplit score columns): the first four
    // softmax warps take the first group, the next four the second, ...; a warp may only touch the
    // TMEM lanes of its quarter (warp % 4).  A group is kCW / 32 sub-slots, one bit-mask word each.
    constexpr int kCW = kTileN / kSplit;           // score columns per thread
    constexpr int kOC = D / kSplit;                // O columns this thread rescales and stores
    constexpr int kOChunk = kOC > 32 ? 32 : kOC;
    const int lq = warp & 3;
    const int quarter = (warp - kSoftmaxWarp0) >> 2;
    const int row = lq * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(lq * 32) << 16;
    const uint32_t tO_mine = tO + lane_off + kOC * quarter;
    const float scale = p.scale_log2;
    int g0 = 0, gu = 0, tq = 0;
    int stored_slot = -1;                          // Q slot holding a staged O tile whose store is in flight
    if (kStageO && warp == kSoftmaxWarp0 && lane == 0) ptx::prefetch_tensormap(&tm_o);
    // The store of the previous tile has had the tile-info loads to read its shared-memory source; the
    // producer may then reuse the slot for the Q tile after next.
    auto release_staged = [&]() {
      if (kStageO && stored_slot >= 0) {
        if (lane == 0) {
          ptx::bulk_wait_group_read0();
          ptx::mbar_arrive(bar(BAR_Q_STORED + stored_slot));
        }
        stored_slot = -1;
      }
    };
    for (int ord = 0;; ++ord) {
      int len_f, len_p;
      const int tile = next_tile_warp(ord, len_f, len_p);
      if (tile >= n_tiles) break;
      const TileInfo ti = tile_info(p, tile, len_f, len_p, nq, nk, eps_shift);
      const int n_full = ti.n_full, total = ti.total, n_steps = ti.n_steps, n_plain = ti.n_plain;
      release_staged();
      T* o_base = static_cast<T*>(p.o) + ti.b_out * p.os[0] + ti.h * p.os[1] +
                  static_cast<int64_t>(ti.qblk) * kTileM * p.os[2];
      uint4* dst = reinterpret_cast<uint4*>(o_base + static_cast<int64_t>(row) * p.os[2] + kOC * quarter);
      float* lse_row = p.lse == nullptr ? nullptr
          : p.lse + (static_cast<int64_t>(ti.b_out) * p.H + ti.h) * p.Sq + ti.qblk * kTileM + row;
      if (n_steps == 0) {                          // nothing attended (in this range): the rows are 0
#pragma unroll
        for (int i = 0; i < kOC / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
        if (lse_row != nullptr && quarter == 0) *lse_row = -INFINITY;
        continue;
      }
      float m = -INFINITY, l = 0.f;                // lines 103-104; l holds this group's partial sum
      bool gave_up = false;
      for (int jj = 0; jj < n_steps; ++jj) {
        const int j = ti.j0 + jj;                  // step of the walk over the lists
        const int g = g0 + jj;                     // steps since the kernel started: buffer and phase
        {
          // S(g) must be complete, and so must O += P.V(g-2), which read the P buffer written below
          // (a barrier that has completed no phase yet passes a wait for parity 1).  Both are asked
          // before either answer is used.
          const uint32_t b_s = bar(BAR_S_FULL + (g & 1)), b_pv = bar(BAR_PV_DONE + (g & 1));
          const uint32_t par_s = (g >> 1) & 1, par_pv = ((g - 2) >> 1) & 1;
          const bool ok_s = ptx::mbar_try_wait(b_s, par_s), ok_pv = ptx::mbar_try_wait(b_pv, par_pv);
          bool mine = true;
          if (!ok_s) mine = ptx::mbar_wait_slow(b_s, par_s, abort_flag);
          if (!ok_pv) mine = ptx::mbar_wait_slow(b_pv, par_pv, abort_flag) && mine;
          // A failed wait (it ran out, or another thread's did) ends the role.  The warp leaves as a whole
          // (warp-wide tensor-memory accesses follow), and it first arrives on the barrier on which the
          // other warp of its rows may be waiting for this step's exchange; that warp finds the abort flag
          // set when it wakes and leaves too.
          if (!__all_sync(0xffffffffu, mine)) {
            ptx::named_bar_arrive(1 + lq, 32 * kSplit);
            gave_up = true;
            break;
          }
        }
        ptx::tc_fence_after();
        // this group's scores of buffer g & 1, and where its P goes
        const uint32_t tS_mine = tmem_base + 128u * (g & 1) + lane_off + kCW * quarter;
        const uint32_t tP_mine = tmem_base + 384u + 64u * (g & 1) + lane_off + (kCW / 2) * quarter;
        const bool masked = j >= n_plain;
        uint32_t w[kCW / 32];
#pragma unroll
        for (int c = 0; c < kCW / 32; ++c) w[c] = 0xffffffffu;
        if (masked) {
          const int u = gu + (j - ti.m0), st = u % kBitStages;
#pragma unroll
          for (int c = 0; c < kCW / 32; ++c) {
            const int ss = quarter * (kCW / 32) + c;           // sub-slot of the step
            const int e = (j << eps_shift) + (ss >> sps_shift);
            const uint32_t word = bits_smem[(st * 4 + ss) * 128 + row];    // stale for a full or padding slot
            w[c] = e < n_full ? 0xffffffffu : (e < total ? word : 0u);
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar(BAR_BITS_EMPTY + st));
        }
        float* xch_mine = xch + ((g & 1) * kSplit + quarter) * 128 + row;
        const float* xch_row = xch + (g & 1) * kSplit * 128 + row;
        auto row_max = [&]() {
          float v = xch_row[0];
#pragma unroll
          for (int q = 1; q < kSplit; ++q) v = fmaxf(v, xch_row[128 * q]);
          return v;
        };

        // One pass against the row's running reference max; a row that has accumulated nothing yet is
        // tried against 0.  The reference only moves (and the pass is redone from the intact scores)
        // when a score exceeds it by more than the threshold, or when a fresh row's largest score
        // lies so far below 0 that P would lose precision.  A row that has seen no attended key at
        // all keeps m = -inf and l = 0.
        const bool fresh = m == -INFINITY;
        const float m_try = fresh ? 0.f : m;
        float m_new = m, alpha = 1.f;
        bool second_pass = true;
        {
          float sum, xmax;
          if (masked) softmax_pass<T, true, kCW>(tS_mine, tP_mine, scale, m_try, w, sum, xmax);
          else        softmax_pass<T, false, kCW>(tS_mine, tP_mine, scale, m_try, w, sum, xmax);
          *xch_mine = xmax;
          ptx::named_bar_sync(1 + lq, 32 * kSplit);
          if (*abort_flag != 0) { gave_up = true; break; }
          const float xrow = row_max();
          const bool seen = xrow > -INFINITY;
          const bool moved = xrow > kRescaleThreshold || (fresh && seen && xrow < kFreshFloor);
          if (!__any_sync(0xffffffffu, moved)) {
            l += sum;
            if (seen) m = m_try;
            second_pass = false;
          } else if (moved) {
            m_new = m_try + xrow;                                   // lines 48 / 50
            alpha = fresh ? 1.f : ex2_approx(-xrow);                // exp2(m - m_new), line 55
          } else if (seen) {
            m_new = m_try;
          }
        }
        if (second_pass) {
          // This step waited for P.V(g-2) and the previous one for P.V(g-3): the barrier of step g-1 is at
          // most one phase behind.
          const bool rescale_o = jj > 0 && __any_sync(0xffffffffu, alpha != 1.f);
          const float sum = second_pass_cold<T, kCW, kOC>(
              tS_mine, tP_mine, tO_mine, scale, m_new == -INFINITY ? 0.f : m_new, alpha, rescale_o,
              bar(BAR_PV_DONE + ((g - 1) & 1)), ((g - 1) >> 1) & 1, abort_flag, w[0], w[kCW / 32 - 1]);
          l = l * alpha + sum;                                      // line 57
          m = m_new;                                                // line 56
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar(BAR_P_FULL + (g & 1)));    // one arrival per softmax warp
      }
      // ---- epilogue of the tile: O / l.  The row sums of the column groups meet in a buffer of their
      // own (the per-step exchange buffers may already be in use by the next tile's first step).
      if (gave_up) break;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(bar(BAR_O_FULL), tq & 1, abort_flag))) {
        ptx::named_bar_arrive(1 + lq, 32 * kSplit);
        break;
      }
      ptx::tc_fence_after();
      float* xl = xch + 2 * kSplit * 128;
      xl[quarter * 128 + row] = l;
      ptx::named_bar_sync(1 + lq, 32 * kSplit);
      if (*abort_flag != 0) break;                 // the other warp of these rows gave up and only arrived
      float l_row = xl[row];
#pragma unroll
      for (int q = 1; q < kSplit; ++q) l_row += xl[128 * q + row];
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;            // line 144, with 0 for an empty row
      if (lse_row != nullptr && quarter == 0)      // m and l are in base 2 (scale folded, line 152)
        *lse_row = l_row > 0.f ? (m + log2f(l_row)) * 0.6931471805599453f : -INFINITY;
      uint32_t ro[kOC];
#pragma unroll
      for (int c = 0; c < kOC / kOChunk; ++c) {
        uint32_t r[kOChunk];
        tmem_load_cols<kOChunk>(tO_mine + c * kOChunk, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < kOChunk; ++i) ro[c * kOChunk + i] = r[i];
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar(BAR_O_FREE));             // O may be overwritten by the next tile
      // A wait that ran out leaves the abort flag set; nothing is written in that case.
      if constexpr (kStageO) {
        // This warp's 32 rows x 128 bytes go to a 4 KB slab of the tile's Q slot (every MMA that read Q
        // completed before O did) in the 128-byte swizzle, then to global memory as one TMA box.
        const int qs = tq & 1;
        const uint32_t slab = sQ + qs * L::kTileBytes + static_cast<uint32_t>(quarter * 4 + lq) * 4096u;
        const bool live = *abort_flag == 0;
#pragma unroll
        for (int i = 0; i < kOC / 8; ++i) {
          const uint32_t a = slab + lane * 128u + (static_cast<uint32_t>(i ^ (lane & 7)) << 4);
          ptx::st_shared_v4(a,
              Fmt<T>::pack2(__uint_as_float(ro[8 * i + 0]) * inv, __uint_as_float(ro[8 * i + 1]) * inv),
              Fmt<T>::pack2(__uint_as_float(ro[8 * i + 2]) * inv, __uint_as_float(ro[8 * i + 3]) * inv),
              Fmt<T>::pack2(__uint_as_float(ro[8 * i + 4]) * inv, __uint_as_float(ro[8 * i + 5]) * inv),
              Fmt<T>::pack2(__uint_as_float(ro[8 * i + 6]) * inv, __uint_as_float(ro[8 * i + 7]) * inv));
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0 && live) {
          ptx::tma_store_4d(&tm_o, slab, kOC * quarter, ti.qblk * kTileM + lq * 32, p.os[1] ? ti.h : 0,
                            p.os[0] ? ti.b_out : 0);                                  // line 146
          ptx::bulk_commit_group();
        }
        stored_slot = qs;
      } else if (*abort_flag == 0) {
#pragma unroll
        for (int i = 0; i < kOC / 8; ++i) {
          uint4 v;
          v.x = Fmt<T>::pack2(__uint_as_float(ro[8 * i + 0]) * inv, __uint_as_float(ro[8 * i + 1]) * inv);
          v.y = Fmt<T>::pack2(__uint_as_float(ro[8 * i + 2]) * inv, __uint_as_float(ro[8 * i + 3]) * inv);
          v.z = Fmt<T>::pack2(__uint_as_float(ro[8 * i + 4]) * inv, __uint_as_float(ro[8 * i + 5]) * inv);
          v.w = Fmt<T>::pack2(__uint_as_float(ro[8 * i + 6]) * inv, __uint_as_float(ro[8 * i + 7]) * inv);
          dst[i] = v;                                               // line 146
        }
      }
      g0 += n_steps;
      gu += max(ti.j1 - ti.m0, 0);
      ++tq;
    }
    release_staged();
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.dev_status != nullptr)
    atomicMax(p.dev_status, SA_DEV_WAIT_EXPIRED);
}

// ---------------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// [B,H,S,D] tensor with element strides st -> 4-D map (d, s, h, b); box = 64 x box_rows.
// Broadcast (stride 0) or singleton dims are given extent 1 and a packed stride.
bool make_map(CUtensorMap* out, const void* base, int dtype, int B, int H, int S, int D,
              const int64_t* st, int box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return false;
  const uint64_t es = 2;
  const uint64_t eh = (st[1] == 0) ? 1 : static_cast<uint64_t>(H);
  const uint64_t eb = (st[0] == 0) ? 1 : static_cast<uint64_t>(B);
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), eh, eb};
  const uint64_t s_row = static_cast<uint64_t>(st[2]) * es;
  const uint64_t s_h = (eh == 1) ? s_row * static_cast<uint64_t>(S) : static_cast<uint64_t>(st[1]) * es;
  const uint64_t s_b = (eb == 1) ? s_h * eh : static_cast<uint64_t>(st[0]) * es;
  cuuint64_t strides[3] = {s_row, s_h, s_b};
  cuuint32_t box[4] = {64u, static_cast<cuuint32_t>(box_rows), 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUtensorMapDataType dt = dtype == SA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool tma_friendly(const void* base, const int64_t* st) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return false;
  if (st[3] != 1) return false;
  if (st[2] <= 0 || st[2] % 8 != 0) return false;
  if (st[1] < 0 || st[1] % 8 != 0 || st[0] < 0 || st[0] % 8 != 0) return false;
  return true;
}

template <typename T, int D>
int launch_inst(const AttnParams& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                const CUtensorMap& mo, cudaStream_t stream) {
  auto kernel = attn_fwd_tc_kernel<T, D>;
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SA_ERR_NO_DEVICE;
  // the opt-in to this much dynamic shared memory is per device and instantiation: done once each
  static std::once_flag once[kMaxDevices];
  static cudaError_t attr_result[kMaxDevices];
  std::call_once(once[info->ordinal], [&] {
    attr_result[info->ordinal] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      static_cast<int>(Smem<D>::dynamic_bytes));
  });
  if (attr_result[info->ordinal] != cudaSuccess) return SA_ERR_CUDA;
  const int n_tiles = (p.Sq / kTileM) * p.B * p.H * p.splits;
  const int grid = n_tiles < info->sm_count ? n_tiles : info->sm_count;    // persistent: one CTA per SM walks the tiles
  if (p.tile_counter != nullptr && cudaMemsetAsync(p.tile_counter, 0, sizeof(int32_t), stream) != cudaSuccess)
    return SA_ERR_CUDA;
  kernel<<<grid, kThreadsTC, Smem<D>::dynamic_bytes, stream>>>(p, mq, mk, mv, mo, n_tiles);
  return cudaGetLastError() == cudaSuccess ? SA_OK : SA_ERR_CUDA;
}

// Split walks: O[row] = sum_s w_s O_s[row] / sum_s w_s with w_s = exp(lse_s - max_s lse_s), the partial
// results being normalised outputs and natural-log sums of the ranges.  One warp per query row; a row no
// range attended comes out as 0 with lse -inf.
template <typename T>
__global__ void __launch_bounds__(256)
merge_splits_kernel(const T* __restrict__ part_o, const float* __restrict__ part_lse, int splits, int B, int H, int Sq,
                    int D, T* __restrict__ o, int64_t os0, int64_t os1, int64_t os2, float* __restrict__ lse) {
  const int64_t rows = static_cast<int64_t>(B) * H * Sq;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int sq = static_cast<int>(row % Sq);
  const int h = static_cast<int>((row / Sq) % H);
  const int b = static_cast<int>(row / (static_cast<int64_t>(Sq) * H));
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_lse[s * rows + row]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float denom = 0.f;
  const int per_lane = D / 32;                     // 2 or 4 consecutive elements
  if (m > -INFINITY) {
    for (int s = 0; s < splits; ++s) {
      const float w = __expf(part_lse[s * rows + row] - m);
      if (w == 0.f) continue;
      denom += w;
      const T* src = part_o + (s * rows + row) * D + lane * per_lane;
      for (int i = 0; i < per_lane; ++i) acc[i] = fmaf(w, static_cast<float>(src[i]), acc[i]);
    }
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  T* dst = o + b * os0 + h * os1 + static_cast<int64_t>(sq) * os2 + lane * per_lane;
  for (int i = 0; i < per_lane; ++i) dst[i] = static_cast<T>(acc[i] * inv);
  if (lse != nullptr && lane == 0) lse[row] = denom > 0.f ? m + __logf(denom) : -INFINITY;
}

}  // namespace

cudaError_t launch_merge_splits(const void* part_o, const float* part_lse, int splits, int dtype, int B, int H, int Sq,
                                int D, void* o, const int64_t* os, float* lse, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(B) * H * Sq;
  const int64_t blocks = (rows * 32 + 255) / 256;
  if (blocks <= 0 || blocks > 0x7fffffffLL || os[3] != 1 || (D != 64 && D != 128)) return cudaErrorInvalidValue;
  if (dtype == SA_DTYPE_BF16)
    merge_splits_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(part_o), part_lse, splits, B, H, Sq, D, static_cast<__nv_bfloat16*>(o), os[0],
        os[1], os[2], lse);
  else if (dtype == SA_DTYPE_F16)
    merge_splits_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const __half*>(part_o), part_lse, splits, B, H, Sq, D, static_cast<__half*>(o), os[0], os[1], os[2],
        lse);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

int attn_tc_supported(const AttnParams& p) {
  if (p.dtype != SA_DTYPE_F16 && p.dtype != SA_DTYPE_BF16) return 0;
  if (p.D != 64 && p.D != 128) return 0;
  if (p.BQ != kTileM) return 0;
  if (p.BK != 32 && p.BK != 64 && p.BK != 128) return 0;
  if (p.Sq % kTileM != 0 || p.Sk % p.BK != 0) return 0;
  if (p.bits == nullptr) return 0;
  if (reinterpret_cast<uintptr_t>(p.bits) % 16 != 0 || p.bits_sb % 4 != 0 || p.bits_sh % 4 != 0) return 0;
  if (!(p.scale_log2 > 0.f) || !(p.scale_log2 < 1e30f)) return 0;
  if (!tma_friendly(p.q, p.qs) || !tma_friendly(p.k, p.ks) || !tma_friendly(p.v, p.vs)) return 0;
  if (reinterpret_cast<uintptr_t>(p.o) % 16 != 0 || p.os[3] != 1 || p.os[2] % 8 != 0 || p.os[1] % 8 != 0 ||
      p.os[0] % 8 != 0)
    return 0;
  return 1;
}

int launch_attn_tc(const AttnParams& p, cudaStream_t stream) {
  if (!attn_tc_supported(p)) return SA_ERR_UNSUPPORTED;
  if (p.splits < 1) return SA_ERR_INVALID_ARGUMENT;
  CUtensorMap mq, mk, mv, mo;
  if (!make_map(&mq, p.q, p.dtype, p.B, p.H, p.Sq, p.D, p.qs, kTileM)) return SA_ERR_CUDA;
  if (!make_map(&mk, p.k, p.dtype, p.B, p.H, p.Sk, p.D, p.ks, p.BK)) return SA_ERR_CUDA;
  if (!make_map(&mv, p.v, p.dtype, p.B, p.H, p.Sk, p.D, p.vs, p.BK)) return SA_ERR_CUDA;
  if (!make_map(&mo, p.o, p.dtype, p.B * p.splits, p.H, p.Sq, p.D, p.os, 32)) return SA_ERR_CUDA;     // one softmax warp's rows
  if (p.dtype == SA_DTYPE_BF16) {
    return p.D == 128 ? launch_inst<__nv_bfloat16, 128>(p, mq, mk, mv, mo, stream)
                      : launch_inst<__nv_bfloat16, 64>(p, mq, mk, mv, mo, stream);
  }
  return p.D == 128 ? launch_inst<__half, 128>(p, mq, mk, mv, mo, stream)
                    : launch_inst<__half, 64>(p, mq, mk, mv, mo, stream);
}

}  // namespace sa
