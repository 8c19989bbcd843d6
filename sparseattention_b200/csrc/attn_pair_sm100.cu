// Stage 2, Blackwell kernel: block-sparse attention forward with TMA + tcgen05 + TMEM.
//
// Replaces sparseattention/sparse_attn_kernel.py:72-146 (kernel) and 10-63 (inner loop)
// for fp16 / bf16, head dim 64 or 128, BLOCK_Q = 128 and BLOCK_K in {32, 64, 128}.
//
// Persistent grid: one CTA per SM (512 threads) runs TWO independent pipelines ("slots"), each working
// through (query block, batch, head) tiles drawn from a device-wide counter.  A tile is one query block
// (128 rows) of one (batch, head); its slot walks the tile's two kv-block lists -- the full list first,
// then the partial list: the order of sparse_attn_kernel.py:113-142 -- in steps of 128 kv rows
// (128 / BLOCK_K listed blocks).  The two slots share nothing but the tensor pipe, the MUFU and the
// tile counter: while the softmax of one slot's step runs, the tensor cores work on the other slot's
// products, and the fixed latencies of a step (barrier waits, tensor-memory loads and stores) of one
// slot are covered by the other slot's exponentials.
//
//   per slot, one warpgroup of helpers (registers cut to 40 each):
//     warp 0   K producer and tile scheduler.  Reads the lists and gathers the listed kv blocks of K into
//              one 128-row, 128-byte-swizzled tile with TMA tile loads whose row coordinate comes from
//              the list, plus the 512-byte bit-mask tiles of the partial blocks (cp.async.bulk from the
//              packed plane of stage 1); loads the Q tile of each query block.
//     warp 1   V producer: the same for V.
//     warp 2   (of slot 0's helpers; it serves both slots) MMA issuer.  S(j) = Q.K(j)^T into the slot's score
//              columns of tensor memory, then -- once the softmax has replaced the scores by P(j) in the same
//              columns -- O += P(j).V(j), then S(j+1), ...: one thread issues them in this order, so the
//              product that reads P(j) is ahead of the product that overwrites it; a slot's "O += P.V, next S"
//              pair is issued back to back, and the pairs of the two slots alternate.
//     others   idle.
//   per slot, one warpgroup of softmax threads (registers raised to 216 each), a thread per query row:
//              scores are exponentiated against the row's running reference max in a single pass (base 2,
//              scale folded as in sparse_attn_kernel.py:152; a row's first scores are tried against 0) and P
//              is held in registers until the row's largest score of the step is known; the reference
//              moves, and the row of O is rescaled in tensor memory, only when a score exceeds it by more
//              than 2^8 (the pass is then redone from the scores, which are still intact).  Steps that
//              contain a partial or padding block apply the bit mask; steps of full blocks do no mask
//              work.  P is rounded to the V dtype (line 61); row sums stay in fp32 (line 57).  Finally
//              O / l is staged in the tile's Q slot and written with TMA stores; a row with no attended key
//              yields 0 (the reference yields NaN, line 53).
//
// Tensor memory (512 columns): slot s has its scores / P at columns 256 s .. 256 s + 127 (P, two values
// per column, over the first 64 of them) and O at 256 s + 128 ..
//
// A step whose last slots run past the end of the lists re-loads the first listed block with an all-zero
// mask word.  Every mbarrier wait is bounded; on expiry the CTA reports SA_DEV_WAIT_EXPIRED, frees its
// tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "ptx_sm100.cuh"
#include "sa_common.cuh"

#ifdef SA_SETMAXNREG
#define SA_COLD __forceinline__
#else
#define SA_COLD __noinline__
#endif

namespace sa {
namespace {

constexpr int kTileM = 128;          // query rows per tile (= BLOCK_Q)
constexpr int kTileN = 128;          // kv rows per MMA step
constexpr int kSlots = 2;            // independent tile pipelines per CTA
constexpr int kThreads = 128 * 2 * kSlots;     // per slot: a helper warpgroup and a softmax warpgroup
constexpr uint32_t kTmemCols = 512;
constexpr int kBitStages = 2;        // masked steps of bit-mask tiles in flight per slot
constexpr int kTileRing = 4;         // tile indices the scheduling warp may be ahead of the slowest role
constexpr uint32_t kPanelBytes = 128u * 128u;   // 128 rows x 64 elements x 2 B
constexpr float kRescaleThreshold = 8.0f;       // log2 units
constexpr float kFreshFloor = -4.0f;            // a row's first scores are taken against 0 if their max is in [-4, 8]
constexpr int kHelperRegs = 40;
constexpr int kSoftmaxRegs = 216;

enum Bar : int {                     // per slot
  BAR_Q_FULL = 0,                    // Q tile landed
  BAR_Q_FREE,                        // 4: the staged O tile has been read out of the Q slot by its stores
  BAR_K_FULL,                        // K tile (and the bit-mask tiles of the step) landed
  BAR_K_EMPTY,                       // K tile consumed by S = Q.K^T
  BAR_V_FULL,
  BAR_V_EMPTY,                       // V tile consumed by O += P.V
  BAR_S_FULL,                        // scores of the step complete (and every earlier product of the slot)
  BAR_P_FULL,                        // 4: P written (and S read) by all softmax warps
  BAR_O_FULL,                        // last O += P.V of a tile complete
  BAR_O_FREE,                        // 4: the epilogue has read O out of tensor memory
  BAR_BITS_EMPTY,                    // kBitStages x 4: bit-mask tiles of a masked step read by the softmax
  BAR_TILE_FULL = BAR_BITS_EMPTY + kBitStages,   // kTileRing: a tile index has been published
  BAR_TILE_EMPTY = BAR_TILE_FULL + kTileRing,    // kTileRing: every other role has read it
  BAR_PER_SLOT = BAR_TILE_EMPTY + kTileRing
};

template <int D>
struct Smem {
  static constexpr uint32_t kTileBytes = kPanelBytes * (D / 64);
  // per slot: Q, K, V tiles, bit-mask stages, list-id rings of the two producers, tile ring
  static constexpr uint32_t off_q = 0;
  static constexpr uint32_t off_k = kTileBytes;
  static constexpr uint32_t off_v = 2 * kTileBytes;
  static constexpr uint32_t off_bits = 3 * kTileBytes;                       // [kBitStages][4 sub-slots][128 rows] u32
  static constexpr uint32_t off_ids = off_bits + kBitStages * 4 * 128 * 4;   // [2 producers][4 steps][4 entries] i32
  static constexpr uint32_t off_ring = off_ids + 2 * 4 * 4 * 4;              // [kTileRing] i32
  static constexpr uint32_t slot_bytes = (off_ring + 4 * kTileRing + 1023) & ~1023u;
  static constexpr uint32_t off_bar = kSlots * slot_bytes;                   // [kSlots][BAR_PER_SLOT] u64
  static constexpr uint32_t off_misc = off_bar + 8 * kSlots * BAR_PER_SLOT;  // TMEM base, abort flag
  static constexpr uint32_t total = off_misc + 16;
  static constexpr uint32_t dynamic_bytes = total + 1024;                    // slack to align the base to 1024 B
};

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

// 32 score columns of one row: x = s*scale - m_ref, masked columns -> -inf (kMasked), P = exp2(x) rounded
// to T into pk, fp32 sum of the unrounded P (lines 54, 57, 61) and max of x.  Two independent accumulator
// pairs, so that consecutive pairs of columns do not wait for one another's result.
template <typename T, bool kMasked>
__device__ __forceinline__ void softmax_chunk(const uint32_t* r, uint32_t w, uint64_t scale2, uint64_t nm2,
                                              uint32_t* pk, uint64_t (&sum2)[2], float (&xmax)[2]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float x0, x1;
    ptx::unpack_f32x2(ptx::fma_f32x2(ptx::pack_u32x2(r[2 * i], r[2 * i + 1]), scale2, nm2), x0, x1);
    if (kMasked) {
      x0 = (w >> (2 * i)) & 1u ? x0 : -INFINITY;                 // line 47
      x1 = (w >> (2 * i + 1)) & 1u ? x1 : -INFINITY;
    }
    xmax[i & 1] = ptx::max3(xmax[i & 1], x0, x1);
#ifdef SA_DBG_NOEXP
    const float p0 = x0 * 0.001f, p1 = x1 * 0.001f;
#else
    const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
#endif
    sum2[i & 1] = ptx::add_f32x2(sum2[i & 1], ptx::pack_f32x2(p0, p1));
    pk[i] = Fmt<T>::pack2(p0, p1);
  }
}

// One pass over the 128 scores of this thread's row, in four chunks of 32 (on masked steps a chunk is
// one 32 x 32 block of the mask for the warp's 32 rows, w[c] its word for this row).  A block that is False
// for all 32 rows costs no arithmetic (P = 0, no exponentials); one that is True for all 32 rows takes the
// mask-free arithmetic.  P stays in registers (pk): the caller writes it once the row's max is known.
template <typename T, bool kMasked>
__device__ __forceinline__ void softmax_pass(uint32_t t_s, float scale, float m_ref, const uint32_t (&w)[4],
                                             uint32_t (&pk)[64], float& sum_out, float& xmax_out) {
  bool dead[4], solid[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    dead[c] = kMasked && __all_sync(0xffffffffu, w[c] == 0u);
    solid[c] = !kMasked || __all_sync(0xffffffffu, w[c] == 0xffffffffu);
  }
  const uint64_t scale2 = ptx::pack_f32x2(scale, scale);
  const uint64_t nm2 = ptx::pack_f32x2(-m_ref, -m_ref);
  uint64_t sum2[2] = {ptx::pack_f32x2(0.f, 0.f), ptx::pack_f32x2(0.f, 0.f)};
  float xmax[2] = {-INFINITY, -INFINITY};
  auto chunk = [&](int c, const uint32_t (&r)[32]) {
    if (dead[c]) {
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[16 * c + i] = 0u;
    } else if (solid[c]) {
      softmax_chunk<T, false>(r, w[c], scale2, nm2, pk + 16 * c, sum2, xmax);
    } else {
      softmax_chunk<T, true>(r, w[c], scale2, nm2, pk + 16 * c, sum2, xmax);
    }
  };
  // two chunks of scores in registers at a time: the loads of the second half travel while the first
  // half is exponentiated
  uint32_t ra[32], rb[32];
  ptx::tmem_ld32(t_s, ra);
  ptx::tmem_ld32(t_s + 32, rb);
  ptx::tmem_ld_wait();
  chunk(0, ra);
  ptx::tmem_ld32(t_s + 64, ra);
  chunk(1, rb);
  ptx::tmem_ld32(t_s + 96, rb);
  ptx::tmem_ld_wait();
  chunk(2, ra);
  chunk(3, rb);
  float s0, s1;
  ptx::unpack_f32x2(ptx::add_f32x2(sum2[0], sum2[1]), s0, s1);
  sum_out = s0 + s1;
  xmax_out = fmaxf(xmax[0], xmax[1]);
}

template <typename T>
__device__ __forceinline__ void store_p(uint32_t t_p, const uint32_t (&pk)[64]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) ptx::tmem_st16(t_p + 16 * c, *reinterpret_cast<const uint32_t(*)[16]>(pk + 16 * c));
}

// The rare second pass of a step, after the reference max of some row of the warp moved, out of line so
// that the hot loop stays small: rescales this thread's row of O by alpha (sparse_attn_kernel.py:58) when
// asked to -- every product so far is complete when the step's scores are, and the next one waits for
// this step's P -- then redoes the pass from the intact scores against m_ref and writes P.  Returns the
// new row sum.  Called by all lanes of a warp (the tensor-memory accesses are warp-wide).
template <typename T, int D>
__device__ SA_COLD float second_pass_cold(uint32_t t_s, uint32_t t_o, float scale, float m_ref, float alpha,
                                               bool rescale_o, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
  if (rescale_o) {
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      ptx::tmem_ld32(t_o + 32 * c, r);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
      ptx::tmem_st32(t_o + 32 * c, r);
    }
  }
  const uint32_t w[4] = {w0, w1, w2, w3};
  uint32_t pk[64];
  float sum, xmax;
  softmax_pass<T, true>(t_s, scale, m_ref, w, pk, sum, xmax);
  store_p<T>(t_s, pk);
  return sum;
}

// Work of one (query block, batch, head) tile, read from the lists.
struct TileInfo {
  int b, h, qblk;
  int n_full, n_part, total, n_steps, n_plain;
};

// Out of line: every role calls it once per tile, and one copy keeps the kernel's code small.
__device__ SA_COLD TileInfo tile_info(const AttnParams& p, int tile, int nq, int nk, int eps_shift) {
  TileInfo t;
  const int bh = tile / nq;
  t.qblk = tile % nq;
  t.b = bh / p.H;
  t.h = bh % p.H;
  int n_full = p.full_lens[t.b * p.fls[0] + t.h * p.fls[1] + static_cast<int64_t>(t.qblk) * p.fls[2]];  // line 107
  int n_part = p.part_lens[t.b * p.pls[0] + t.h * p.pls[1] + static_cast<int64_t>(t.qblk) * p.pls[2]];  // line 127
  t.n_full = min(max(n_full, 0), nk);
  t.n_part = min(max(n_part, 0), nk);
  t.total = t.n_full + t.n_part;
  t.n_steps = (t.total + (1 << eps_shift) - 1) >> eps_shift;
  t.n_plain = t.n_full >> eps_shift;   // leading steps made of full blocks only
  return t;
}

__device__ __forceinline__ void setmaxnreg_dec() {
#ifdef SA_SETMAXNREG
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHelperRegs));
#endif
}
__device__ __forceinline__ void setmaxnreg_inc() {
#ifdef SA_SETMAXNREG
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
#endif
}


template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 1)
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
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_misc + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wg = warp >> 2;                         // warpgroups 0, 1: helpers of slot 0, 1; 2, 3: softmax of slot 0, 1
  const int slot = wg & 1;
  const bool is_softmax = wg >= kSlots;
  const int wq = warp & 3;                          // warp within its warpgroup (= tensor-memory lane quarter)

  uint8_t* sl_smem = smem + slot * L::slot_bytes;
  const uint32_t sl_base = sbase + slot * L::slot_bytes;
  const uint32_t sQ = sl_base + L::off_q, sK = sl_base + L::off_k, sV = sl_base + L::off_v;
  const uint32_t sBits = sl_base + L::off_bits;
  const uint32_t* bits_smem = reinterpret_cast<const uint32_t*>(sl_smem + L::off_bits);
  volatile int* tile_ring = reinterpret_cast<volatile int*>(sl_smem + L::off_ring);
  auto bar = [&](int i) { return sbase + L::off_bar + 8u * static_cast<uint32_t>(slot * BAR_PER_SLOT + i); };

  const int nq = p.Sq / kTileM;
  const int nk = p.Sk / p.BK;
  // BLOCK_K is 32, 64 or 128: list entries per step (4, 2, 1) and 32-column sub-slots per entry
  // (1, 2, 4) are powers of two, so the per-step index arithmetic is shifts.
  const int eps_shift = p.BK == 32 ? 2 : (p.BK == 64 ? 1 : 0);
  const int sps_shift = 2 - eps_shift;
  const int eps = 1 << eps_shift;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
      auto b = [&](int i) { return sbase + L::off_bar + 8u * static_cast<uint32_t>(s * BAR_PER_SLOT + i); };
      ptx::mbar_init(b(BAR_Q_FULL), 1);
      ptx::mbar_init(b(BAR_Q_FREE), 4);
      ptx::mbar_init(b(BAR_K_FULL), 1);
      ptx::mbar_init(b(BAR_K_EMPTY), 1);
      ptx::mbar_init(b(BAR_V_FULL), 1);
      ptx::mbar_init(b(BAR_V_EMPTY), 1);
      ptx::mbar_init(b(BAR_S_FULL), 1);
      ptx::mbar_init(b(BAR_P_FULL), 4);                   // one arrival per softmax warp
      ptx::mbar_init(b(BAR_O_FULL), 1);
      ptx::mbar_init(b(BAR_O_FREE), 4);
      for (int i = 0; i < kBitStages; ++i) ptx::mbar_init(b(BAR_BITS_EMPTY + i), 4);
      for (int i = 0; i < kTileRing; ++i) {
        ptx::mbar_init(b(BAR_TILE_FULL + i), 1);
        ptx::mbar_init(b(BAR_TILE_EMPTY + i), 2 + 4);     // V producer, MMA issuer, softmax warps
      }
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
  const uint32_t tS = tmem_base + 256u * slot;      // scores, then P over the first 64 columns
  const uint32_t tO = tS + 128u;

  // Every role of a slot walks the same sequence of tiles and keeps the same running counts -- steps done
  // (g), masked steps done (gu), non-empty tiles done (tq) -- from which barrier phases follow; nothing
  // is reset between tiles.  The sequence of slot s of CTA c starts at tile 2 c + s; the slot's K producer
  // draws each further tile from a device-wide counter (or, without one, steps by twice the grid size) and
  // publishes it to the slot's other roles through a small ring in shared memory; an index >= n_tiles ends
  // every role's loop.  Ordinal `ord` of the sequence lives in ring slot ord % kTileRing.
  // A wait that fails (it ran out, or another thread's did) ends the role's loop; the decision is taken
  // warp-wide so that no lane is left alone in a warp-wide tensor-memory instruction.
  auto read_tile_warp = [&](int ord) -> int {       // a whole warp; lane 0 waits, reads and hands the slot back
    int t = n_tiles;
    if (lane == 0) {
      const int rs = ord % kTileRing;
      if (ptx::mbar_wait(bar(BAR_TILE_FULL + rs), (ord / kTileRing) & 1, abort_flag)) {
        t = tile_ring[rs];
        ptx::mbar_arrive(bar(BAR_TILE_EMPTY + rs));
      }
    }
    return __shfl_sync(0xffffffffu, t, 0);
  };

  if (!is_softmax) {
    setmaxnreg_dec();
    if (wq < 2) {
      // ------------------------------------------------------------------ producers
      // Warp 0 of the warpgroup gathers Q, the K tiles and the bit-mask tiles, warp 1 the V tiles.  The
      // whole warp runs the loop: lane 0 waits for the free stage and arms its barrier, lanes 0-7 each
      // issue one TMA box, lanes 0-3 fetch the list entries of a step.
      const bool is_k = wq == 0;
      const CUtensorMap* tm = is_k ? &tm_k : &tm_v;
      if (lane == 0) {
        ptx::prefetch_tensormap(tm);
        if (is_k) ptx::prefetch_tensormap(&tm_q);
      }
      const uint32_t s_tile = is_k ? sK : sV;
      const int bar_full = is_k ? BAR_K_FULL : BAR_V_FULL, bar_empty = is_k ? BAR_K_EMPTY : BAR_V_EMPTY;
      const uint32_t blk_bytes = static_cast<uint32_t>(p.BK) * 128u;
      constexpr int kPanels = D / 64;
      const int c_of_lane = lane / kPanels, pnl_of_lane = lane % kPanels;
      const bool has_box = c_of_lane < eps;
      bool bad_index = false;
      bool ok = true;
      int g = 0, gu = 0, tq = 0;
      const uint32_t s_ids = sl_base + L::off_ids + static_cast<uint32_t>(wq) * 64u;
      const volatile int* ids_ring = reinterpret_cast<const volatile int*>(sl_smem + L::off_ids + wq * 64);
      // lane 0 of the K producer publishes tile `t` as ordinal `ord` of the slot's sequence
      auto publish = [&](int ord, int t) {
        const int rs = ord % kTileRing;
        if (ord >= kTileRing) ok = ptx::mbar_wait(bar(BAR_TILE_EMPTY + rs), (ord / kTileRing - 1) & 1, abort_flag);
        tile_ring[rs] = (ok && *abort_flag == 0) ? t : n_tiles;
        ptx::mbar_arrive(bar(BAR_TILE_FULL + rs));
      };
      int ord = 0;
#ifdef SA_DBG_ONESLOT
      constexpr int kActive = 1;
      int tile = slot == 0 ? static_cast<int>(blockIdx.x) : n_tiles;
#else
      constexpr int kActive = kSlots;
      int tile = static_cast<int>(blockIdx.x) * kSlots + slot;
#endif
      if (is_k) { if (lane == 0) publish(0, tile); } else { tile = read_tile_warp(0); }
      while (tile < n_tiles && ok) {
        // The next tile is drawn now and published after this one's loads are issued: the answer of
        // the atomic is not waited for until then.
        int drawn = 0;
        if (is_k && lane == 0)
          drawn = p.tile_counter != nullptr ? atomicAdd(p.tile_counter, 1) : 0;
        const TileInfo ti = tile_info(p, tile, nq, nk, eps_shift);
        const int b = ti.b, h = ti.h, qblk = ti.qblk, n_full = ti.n_full, total = ti.total, n_steps = ti.n_steps,
                  n_plain = ti.n_plain;
        if (total != 0) {
          if (is_k) {                                 // Q tile of this query block
            if (lane == 0) {
              // the Q slot held the previous tile's staged O: its stores must have read it
              if (tq >= 1) ok = ptx::mbar_wait(bar(BAR_Q_FREE), (tq - 1) & 1, abort_flag);
              if (ok) {
                const int qb = p.qs[0] ? b : 0, qh = p.qs[1] ? h : 0;
                ptx::mbar_arrive_expect_tx(bar(BAR_Q_FULL), L::kTileBytes);
#pragma unroll
                for (int pnl = 0; pnl < D / 64; ++pnl)
                  ptx::tma_load_4d(sQ + pnl * kPanelBytes, &tm_q, bar(BAR_Q_FULL), pnl * 64, qblk * kTileM, qh, qb);
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
            if (lane < eps && j < n_steps) {
              const int e = (j << eps_shift) + lane;
              const int ee = e < total ? e : 0;         // slots past the end re-load the first listed block
              const int32_t* src = ee < n_full ? fids + ee * p.fis[3] : pids + (ee - n_full) * p.pis[3];   // line 33
              ptx::cp_async_4(s_ids + static_cast<uint32_t>((j & 3) * 4 + lane) * 4u, src);
            }
            ptx::cp_async_commit();
          };
          __syncwarp();                                     // every lane has read the previous tile's last entries
          fetch_ids(0);
          fetch_ids(1);
          for (int j = 0; j < n_steps && ok; ++j, ++g) {
            fetch_ids(j + 2);
            ptx::cp_async_wait<2>();                        // the group of step j has landed
            __syncwarp();
            const uint32_t full_bar = bar(bar_full);
            // The bit-mask tiles of the partial blocks of step j land on the K tile's barrier: once
            // S(j) is complete the softmax finds them in shared memory without a wait of its own.
            const bool with_bits = is_k && j >= n_plain;
            const int u = gu + (j - n_plain), bst = u % kBitStages;
            uint32_t tx_bytes = L::kTileBytes;
            if (with_bits) {
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int e = (j << eps_shift) + (c >> sps_shift);
                tx_bytes += (e >= n_full && e < total) ? 512u : 0u;
              }
            }
            if (lane == 0) {
              if (g > 0) ok = ptx::mbar_wait(bar(bar_empty), (g - 1) & 1, abort_flag);
              if (ok && with_bits && u >= kBitStages)
                ok = ptx::mbar_wait(bar(BAR_BITS_EMPTY + bst), (u / kBitStages - 1) & 1, abort_flag);
#ifdef SA_DBG_NOLOAD
              if (ok) { if (g == 0) ptx::mbar_arrive_expect_tx(full_bar, L::kTileBytes); else ptx::mbar_arrive(full_bar); }
#else
              if (ok) ptx::mbar_arrive_expect_tx(full_bar, tx_bytes);
#endif
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            int id_c = ids_ring[(j & 3) * 4 + (c_of_lane & 3)];
            if (static_cast<unsigned>(id_c) >= static_cast<unsigned>(nk)) { bad_index = bad_index || has_box; id_c = 0; }
#ifdef SA_DBG_NOLOAD
            if (g > 0) continue;
#endif
            if (ok && has_box)
              ptx::tma_load_4d(s_tile + pnl_of_lane * kPanelBytes + c_of_lane * blk_bytes, tm, full_bar,
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
          }
          gu += n_steps - n_plain;
          ++tq;
        }
        ++ord;
        if (is_k) {
          if (lane == 0) {
            if (p.tile_counter != nullptr) drawn += static_cast<int>(gridDim.x) * kActive;
            else drawn = (ord * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x)) * kActive + slot;
            if (drawn < 0 || drawn > n_tiles) drawn = n_tiles;
            publish(ord, drawn);
          }
          tile = __shfl_sync(0xffffffffu, drawn, 0);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        } else {
          tile = read_tile_warp(ord);
        }
      }
      if (is_k && __any_sync(0xffffffffu, bad_index) && lane == 0 && p.dev_status != nullptr)
        atomicMax(p.dev_status, SA_DEV_BAD_INDEX);
      __syncwarp();
    } else if (warp == 2) {
      // ------------------------------------------------------------------ MMA issuer (one thread, both slots)
      // Per slot: S(g) = Q.K(g)^T (line 40), then O += P(g).V(g) (line 61) once the softmax has put P(g)
      // where the scores were, then S(g+1), ...  One thread issues the products of both slots, a slot's
      // "O += P.V, next S" pair back to back: the tensor pipe runs them in issue order, so while one
      // slot's pair executes the other slot's softmax runs, and the two slots settle half a step apart
      // instead of competing for the tensor pipe and the MUFU at the same moments.  The thread never
      // blocks on one slot: it polls what each slot needs next.
      if (lane == 0) {
        constexpr uint32_t idesc_s = ptx::umma_idesc_f16(Fmt<T>::umma, kTileM, kTileN, 0);
        constexpr uint32_t idesc_o = ptx::umma_idesc_f16(Fmt<T>::umma, kTileM, D, 1);
        enum Need : int { NEED_TILE, NEED_Q, NEED_S, NEED_PV, FINISHED };
        struct SlotState {
          int need, ord, j, g, tq, n_steps;
          uint32_t bars, tS, tO, dq_lo, dk_lo, dv_lo;
        } st[kSlots];
        uint32_t d_hi = 0, dv_hi = 0;
        for (int s = 0; s < kSlots; ++s) {
          const uint32_t base_s = sbase + s * L::slot_bytes;
          const uint64_t dq = ptx::umma_desc_sw128(base_s + L::off_q, 16u);
          const uint64_t dv = ptx::umma_desc_sw128(base_s + L::off_v, kPanelBytes);
          d_hi = static_cast<uint32_t>(dq >> 32);
          dv_hi = static_cast<uint32_t>(dv >> 32);
          st[s] = SlotState{NEED_TILE, 0, 0, 0, 0, 0,
                            sbase + L::off_bar + 8u * static_cast<uint32_t>(s * BAR_PER_SLOT),
                            tmem_base + 256u * s, tmem_base + 256u * s + 128u,
                            static_cast<uint32_t>(dq),
                            static_cast<uint32_t>(ptx::umma_desc_sw128(base_s + L::off_k, 16u)),
                            static_cast<uint32_t>(dv)};
        }
        const uint64_t t0 = ptx::global_timer_ns();
        uint64_t last_progress = t0;
        uint32_t idle = 0;
        int finished = 0;
        while (finished < kSlots) {
          bool progressed = false;
#pragma unroll
          for (int s = 0; s < kSlots; ++s) {
            SlotState& x = st[s];
            auto sb = [&](int i) { return x.bars + 8u * static_cast<uint32_t>(i); };
            if (x.need == NEED_TILE) {
              const int rs = x.ord % kTileRing;
              if (!ptx::mbar_try_wait(sb(BAR_TILE_FULL + rs), (x.ord / kTileRing) & 1)) continue;
              const int tile = reinterpret_cast<volatile int*>(smem + s * L::slot_bytes + L::off_ring)[rs];
              ptx::mbar_arrive(sb(BAR_TILE_EMPTY + rs));
              progressed = true;
              if (tile >= n_tiles) { x.need = FINISHED; ++finished; continue; }
              const TileInfo ti = tile_info(p, tile, nq, nk, eps_shift);
              ++x.ord;
              if (ti.total == 0) continue;
              x.n_steps = ti.n_steps;
              x.j = 0;
              x.need = NEED_Q;
            }
            if (x.need == NEED_Q) {
              if (!ptx::mbar_try_wait(sb(BAR_Q_FULL), x.tq & 1)) continue;
              x.need = NEED_S;
              progressed = true;
            }
            if (x.need == NEED_PV) {
              if (!ptx::mbar_try_wait(sb(BAR_P_FULL), x.g & 1)) continue;
              if (!ptx::mbar_try_wait(sb(BAR_V_FULL), x.g & 1)) continue;
              // the first product of a tile overwrites O: the previous tile's epilogue must have read it
              if (x.j == 0 && x.tq >= 1 && !ptx::mbar_try_wait(sb(BAR_O_FREE), (x.tq - 1) & 1)) continue;
              ptx::tc_fence_after();
              if (x.j == 0) {
#pragma unroll
                for (int kk = 0; kk < kTileN / 16; ++kk) {
                  if (kk == 0) ptx::mma_ts_lo<false>(x.tO, x.tS + kk * 8u, x.dv_lo + kk * 128u, dv_hi, idesc_o);
                  else         ptx::mma_ts_lo<true>(x.tO, x.tS + kk * 8u, x.dv_lo + kk * 128u, dv_hi, idesc_o);
                }
              } else {
#pragma unroll
                for (int kk = 0; kk < kTileN / 16; ++kk)
                  ptx::mma_ts_lo<true>(x.tO, x.tS + kk * 8u, x.dv_lo + kk * 128u, dv_hi, idesc_o);
              }
              ptx::mma_commit(sb(BAR_V_EMPTY));
              ++x.j;
              ++x.g;
              progressed = true;
              if (x.j == x.n_steps) {
                ptx::mma_commit(sb(BAR_O_FULL));
                ++x.tq;
                x.need = NEED_TILE;
                continue;
              }
              x.need = NEED_S;
            }
            if (x.need == NEED_S) {
              if (!ptx::mbar_try_wait(sb(BAR_K_FULL), x.g & 1)) continue;
              ptx::tc_fence_after();
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk) {
                constexpr uint32_t kPanelStep = kPanelBytes >> 4;
                const uint32_t off = (kk / 4) * kPanelStep + (kk % 4) * 2u;      // (panel, 32-byte K slice) >> 4
                if (kk == 0) ptx::mma_ss_lo<false>(x.tS, x.dq_lo + off, x.dk_lo + off, d_hi, idesc_s);
                else         ptx::mma_ss_lo<true>(x.tS, x.dq_lo + off, x.dk_lo + off, d_hi, idesc_s);
              }
              ptx::mma_commit(sb(BAR_K_EMPTY));
              ptx::mma_commit(sb(BAR_S_FULL));
              x.need = NEED_PV;
              progressed = true;
            }
          }
          // bounded: no progress on either slot for the wait limit (or another role gave up) ends the loop
          if (progressed) {
            idle = 0;
          } else if ((++idle & 0x3ffu) == 0u) {
            const uint64_t now = ptx::global_timer_ns();
            if (idle == 0x400u) last_progress = now;
            if (*abort_flag != 0) break;
            if (now - last_progress > ptx::kWaitLimitNs) { *abort_flag = 1; break; }
          }
        }
      }
      __syncwarp();
    }
    // the other warps of the helper warpgroups have nothing to do
  } else {
    setmaxnreg_inc();
    // ------------------------------------------------------------------ softmax: thread = query row
    const int row = wq * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tS_mine = tS + lane_off, tO_mine = tO + lane_off;
    const float scale = p.scale_log2;
    int g = 0, gu = 0, tq = 0;
    bool staged = false;                             // a staged O tile's stores are in flight
    if (wq == 0 && lane == 0) ptx::prefetch_tensormap(&tm_o);
    // The stores of the previous tile have had the tile-info loads to read their shared-memory source; the
    // producer may then load the next Q tile into the slot.
    auto release_staged = [&]() {
      if (staged) {
        if (lane == 0) {
          ptx::bulk_wait_group_read0();
          ptx::mbar_arrive(bar(BAR_Q_FREE));
        }
        staged = false;
      }
    };
    bool ok = true;
    for (int ord = 0; ok; ++ord) {
      const int tile = read_tile_warp(ord);
      if (tile >= n_tiles) break;
      const TileInfo ti = tile_info(p, tile, nq, nk, eps_shift);
      const int n_full = ti.n_full, total = ti.total, n_steps = ti.n_steps, n_plain = ti.n_plain;
      float* lse_row = p.lse == nullptr ? nullptr
          : p.lse + (static_cast<int64_t>(ti.b) * p.H + ti.h) * p.Sq + ti.qblk * kTileM + row;
      if (total == 0) {                            // nothing attended: the rows are 0
        T* o_row = static_cast<T*>(p.o) + ti.b * p.os[0] + ti.h * p.os[1] +
                   (static_cast<int64_t>(ti.qblk) * kTileM + row) * p.os[2];
        uint4* dst = reinterpret_cast<uint4*>(o_row);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
        if (lse_row != nullptr) *lse_row = -INFINITY;
        continue;
      }
      release_staged();
      float m = -INFINITY, l = 0.f;                // lines 103-104
      for (int j = 0; j < n_steps; ++j, ++g) {
        // S(g) complete; every earlier product of the slot is complete with it, so O is at rest
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(bar(BAR_S_FULL), g & 1, abort_flag));
        if (!ok) break;
        ptx::tc_fence_after();
#ifdef SA_DBG_NOSOFTMAX
        if (j >= n_plain) { __syncwarp(); if (lane == 0) ptx::mbar_arrive(bar(BAR_BITS_EMPTY + (gu + (j - n_plain)) % kBitStages)); }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar(BAR_P_FULL));
        continue;
#endif
        const bool masked = j >= n_plain;
        uint32_t w[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        if (masked) {
          const int u = gu + (j - n_plain), st = u % kBitStages;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int e = (j << eps_shift) + (c >> sps_shift);
            const uint32_t word = bits_smem[(st * 4 + c) * 128 + row];    // stale for a full or padding slot
            w[c] = e < n_full ? 0xffffffffu : (e < total ? word : 0u);
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar(BAR_BITS_EMPTY + st));
        }
        // One pass against the row's running reference max; a row that has accumulated nothing yet is
        // tried against 0.  The reference only moves (and the pass is redone from the intact scores)
        // when a score exceeds it by more than the threshold, or when a fresh row's largest score
        // lies so far below 0 that P would lose precision.  A row that has seen no attended key at
        // all keeps m = -inf and l = 0.
        const bool fresh = m == -INFINITY;
        const float m_try = fresh ? 0.f : m;
        float m_new = m, alpha = 1.f;
        bool moved_any;
        {
          uint32_t pk[64];
          float sum, xrow;
          if (masked) softmax_pass<T, true>(tS_mine, scale, m_try, w, pk, sum, xrow);
          else        softmax_pass<T, false>(tS_mine, scale, m_try, w, pk, sum, xrow);
          const bool seen = xrow > -INFINITY;
          const bool moved = xrow > kRescaleThreshold || (fresh && seen && xrow < kFreshFloor);
          moved_any = __any_sync(0xffffffffu, moved);
          if (!moved_any) {
            store_p<T>(tS_mine, pk);
            l += sum;
            if (seen) m = m_try;
          } else if (moved) {
            m_new = m_try + xrow;                                   // lines 48 / 50
            alpha = fresh ? 1.f : ex2_approx(-xrow);                // exp2(m - m_new), line 55
          } else if (seen) {
            m_new = m_try;
          }
        }
        if (moved_any) {
          const bool rescale_o = j > 0 && __any_sync(0xffffffffu, alpha != 1.f);
          const float sum = second_pass_cold<T, D>(tS_mine, tO_mine, scale, m_new == -INFINITY ? 0.f : m_new, alpha,
                                                   rescale_o, w[0], w[1], w[2], w[3]);
          l = l * alpha + sum;                                      // line 57
          m = m_new;                                                // line 56
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar(BAR_P_FULL));           // one arrival per softmax warp
      }
      if (!ok) break;
      // ---- epilogue of the tile: O / l
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(bar(BAR_O_FULL), tq & 1, abort_flag));
      if (!ok) break;
      ptx::tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;                    // line 144, with 0 for an empty row
      if (lse_row != nullptr)                      // m and l are in base 2 (scale folded, line 152)
        *lse_row = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
      // This warp's 32 rows go to a 4 KB slab per 64-column panel of the tile's Q slot (every product that
      // read Q is complete) in the 128-byte swizzle, then to global memory as one TMA box per panel.
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld32(tO_mine + 32 * c, r);
        ptx::tmem_ld_wait();
        if (c == D / 32 - 1) {
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar(BAR_O_FREE));         // O may be overwritten by the next tile
        }
        const uint32_t slab = sQ + static_cast<uint32_t>(c / 2) * kPanelBytes + static_cast<uint32_t>(wq) * 4096u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int unit = (c & 1) * 4 + i;
          const uint32_t a = slab + lane * 128u + (static_cast<uint32_t>(unit ^ (lane & 7)) << 4);
          ptx::st_shared_v4(a,
              Fmt<T>::pack2(__uint_as_float(r[8 * i + 0]) * inv, __uint_as_float(r[8 * i + 1]) * inv),
              Fmt<T>::pack2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv),
              Fmt<T>::pack2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv),
              Fmt<T>::pack2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv));
        }
      }
      ptx::fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        if (*abort_flag == 0) {                    // a wait that ran out leaves the flag set; nothing is written then
#pragma unroll
          for (int pnl = 0; pnl < D / 64; ++pnl)
            ptx::tma_store_4d(&tm_o, sQ + pnl * kPanelBytes + static_cast<uint32_t>(wq) * 4096u, 64 * pnl,
                              ti.qblk * kTileM + wq * 32, p.os[1] ? ti.h : 0, p.os[0] ? ti.b : 0);   // line 146
        }
        ptx::bulk_commit_group();
      }
      staged = true;
      gu += n_steps - n_plain;
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
  const int n_tiles = (p.Sq / kTileM) * p.B * p.H;
#ifdef SA_DBG_ONESLOT
  const int want = n_tiles;
#else
  const int want = (n_tiles + kSlots - 1) / kSlots;
#endif
  const int grid = want < info->sm_count ? want : info->sm_count;    // persistent: one CTA per SM walks the tiles
  if (p.tile_counter != nullptr && cudaMemsetAsync(p.tile_counter, 0, sizeof(int32_t), stream) != cudaSuccess)
    return SA_ERR_CUDA;
  kernel<<<grid, kThreads, Smem<D>::dynamic_bytes, stream>>>(p, mq, mk, mv, mo, n_tiles);
  return cudaGetLastError() == cudaSuccess ? SA_OK : SA_ERR_CUDA;
}

}  // namespace

int attn_tc2_supported(const AttnParams& p) {
  if (p.dtype != SA_DTYPE_F16 && p.dtype != SA_DTYPE_BF16) return 0;
  if (p.D != 64 && p.D != 128) return 0;
  if (p.BQ != kTileM) return 0;
  if (p.BK != 32 && p.BK != 64 && p.BK != 128) return 0;
  if (p.Sq % kTileM != 0 || p.Sk % p.BK != 0) return 0;
  if (p.bits == nullptr) return 0;
  if (reinterpret_cast<uintptr_t>(p.bits) % 16 != 0 || p.bits_sb % 4 != 0 || p.bits_sh % 4 != 0) return 0;
  if (!(p.scale_log2 > 0.f) || !(p.scale_log2 < 1e30f)) return 0;
  if (!tma_friendly(p.q, p.qs) || !tma_friendly(p.k, p.ks) || !tma_friendly(p.v, p.vs)) return 0;
  if (!tma_friendly(p.o, p.os)) return 0;
  if (static_cast<long long>(p.Sq / kTileM) * p.B * p.H > 0x3fffffffLL) return 0;
  return 1;
}

int launch_attn_tc2(const AttnParams& p, cudaStream_t stream) {
  if (!attn_tc2_supported(p)) return SA_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv, mo;
  if (!make_map(&mq, p.q, p.dtype, p.B, p.H, p.Sq, p.D, p.qs, kTileM)) return SA_ERR_CUDA;
  if (!make_map(&mk, p.k, p.dtype, p.B, p.H, p.Sk, p.D, p.ks, p.BK)) return SA_ERR_CUDA;
  if (!make_map(&mv, p.v, p.dtype, p.B, p.H, p.Sk, p.D, p.vs, p.BK)) return SA_ERR_CUDA;
  if (!make_map(&mo, p.o, p.dtype, p.B, p.H, p.Sq, p.D, p.os, 32)) return SA_ERR_CUDA;     // one softmax warp's rows
  if (p.dtype == SA_DTYPE_BF16) {
    return p.D == 128 ? launch_inst<__nv_bfloat16, 128>(p, mq, mk, mv, mo, stream)
                      : launch_inst<__nv_bfloat16, 64>(p, mq, mk, mv, mo, stream);
  }
  return p.D == 128 ? launch_inst<__half, 128>(p, mq, mk, mv, mo, stream)
                    : launch_inst<__half, 64>(p, mq, mk, mv, mo, stream);
}

}  // namespace sa
