// Stage 2, Blackwell kernel: block-sparse attention forward with TMA + tcgen05 + TMEM.
//
// Replaces sparseattention/sparse_attn_kernel.py:72-146 (kernel) and 10-63 (inner loop)
// for fp16 / bf16, head dim 64 or 128, BLOCK_Q = 128 and BLOCK_K in {32, 64, 128}.
//
// One CTA owns one query block (128 rows) of one (batch, head); two CTAs share an SM so
// that the tensor pipe of one overlaps the softmax of the other.  Per CTA:
//
//   warp 0    producer.  Reads the two kv-block id lists of the query block (full list first,
//             then the partial list: the order of sparse_attn_kernel.py:113-142) and, for each
//             step of 128 kv rows, gathers 128/BLOCK_K listed kv blocks of K and of V into one
//             128-row, 128-byte-swizzled shared-memory tile with TMA tile loads whose row
//             coordinate comes from the list, plus the 512-byte bit-mask tiles of the
//             partial blocks (cp.async.bulk from the packed plane of stage 1).
//   warp 1    MMA issuer.  S = Q.K^T (tcgen05.mma, both operands in shared memory, fp32
//             accumulator in tensor memory), then O += P.V with P read from tensor memory.
//   warps 2-5 softmax, one thread per query row.  Reads S from tensor memory, applies the bit
//             mask on steps that contain a partial or padding block, keeps the running max /
//             sum in fp32 in base 2 (scale folded as in sparse_attn_kernel.py:152), writes P
//             (rounded to the V dtype, line 61) over S in tensor memory, rescales O in tensor
//             memory only when the running max grew by more than 2^8, and finally writes
//             O / l.  A row with no attended key yields 0 (the reference yields NaN, line 53).
//
// Steps made only of full blocks skip all mask work.  A step whose last slots run past the
// end of the lists re-loads the first listed block with an all-zero mask word.
// Every mbarrier wait is bounded; on expiry the CTA reports SA_DEV_WAIT_EXPIRED, frees its
// tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"
#include "sa_common.cuh"

namespace sa {
namespace {

constexpr int kTileM = 128;          // query rows per CTA (= BLOCK_Q)
constexpr int kTileN = 128;          // kv rows per MMA step
constexpr int kThreadsTC = 320;         // producer warp, MMA warp, 8 softmax warps
constexpr uint32_t kTmemCols = 256;  // S/P: columns [0,128), O: [128, 128+D)
constexpr uint32_t kPanelBytes = 128u * 128u;   // 128 rows x 64 elements x 2 B
constexpr float kRescaleThreshold = 8.0f;       // log2 units

enum Bar : int {
  BAR_Q = 0, BAR_K_FULL, BAR_K_EMPTY, BAR_V_FULL, BAR_V_EMPTY, BAR_S_FULL, BAR_P_FULL, BAR_O_FULL,
  BAR_BITS_FULL0, BAR_BITS_FULL1, BAR_BITS_EMPTY0, BAR_BITS_EMPTY1, BAR_COUNT
};

template <int D>
struct Smem {
  static constexpr uint32_t kTileBytes = kPanelBytes * (D / 64);
  static constexpr uint32_t off_q = 0;
  static constexpr uint32_t off_k = kTileBytes;
  static constexpr uint32_t off_v = 2 * kTileBytes;
  static constexpr uint32_t off_bits = 3 * kTileBytes;          // [2 stages][4 sub-slots][128 rows] u32
  static constexpr uint32_t off_bar = off_bits + 2 * 4 * 128 * 4;
  static constexpr uint32_t off_misc = off_bar + 8 * 16;
  static constexpr uint32_t off_xch = off_misc + 16;             // [2 parities][2 halves][128 rows] f32
  static constexpr uint32_t total = off_xch + 2 * 2 * 128 * 4;
  static constexpr uint32_t dynamic_bytes = total + 1024;       // slack to align the base to 1024 B
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


// One pass over this thread's 64 score columns (two TMEM loads of 32): x = s*scale - m_ref,
// masked columns -> -inf, P = exp2(x) rounded to T and written over the first 32 columns of the
// thread's own score range, fp32 row sum of the unrounded P (lines 54, 57, 61) and max of x.
template <typename T, bool kMasked>
__device__ __forceinline__ void softmax_pass(uint32_t t_half, float scale, float m_ref, uint32_t w0, uint32_t w1,
                                             float& sum_out, float& xmax_out) {
  uint32_t r0[32], r1[32];
  ptx::tmem_ld32(t_half, r0);
  ptx::tmem_ld32(t_half + 32, r1);
  ptx::tmem_ld_wait();
  const uint64_t scale2 = ptx::pack_f32x2(scale, scale);
  const uint64_t nm2 = ptx::pack_f32x2(-m_ref, -m_ref);
  uint64_t sum2 = ptx::pack_f32x2(0.f, 0.f);
  float xmax = -INFINITY;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t a = c == 0 ? r0[2 * i] : r1[2 * i];
      const uint32_t b = c == 0 ? r0[2 * i + 1] : r1[2 * i + 1];
      float x0, x1;
      ptx::unpack_f32x2(ptx::fma_f32x2(ptx::pack_u32x2(a, b), scale2, nm2), x0, x1);
      if (kMasked) {
        const uint32_t w = c == 0 ? w0 : w1;
        x0 = (w >> (2 * i)) & 1u ? x0 : -INFINITY;                 // line 47
        x1 = (w >> (2 * i + 1)) & 1u ? x1 : -INFINITY;
      }
      xmax = ptx::max3(xmax, x0, x1);
      const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
      sum2 = ptx::add_f32x2(sum2, ptx::pack_f32x2(p0, p1));
      pk[i] = Fmt<T>::pack2(p0, p1);
    }
    ptx::tmem_st16(t_half + c * 16, pk);
  }
  float s0, s1;
  ptx::unpack_f32x2(sum2, s0, s1);
  sum_out = s0 + s1;
  xmax_out = xmax;
}

// Max of the raw (masked) scores of this thread's 64 columns.
template <bool kMasked>
__device__ __forceinline__ void max_pass(uint32_t t_half, uint32_t w0, uint32_t w1, float& smax_out) {
  uint32_t r0[32], r1[32];
  ptx::tmem_ld32(t_half, r0);
  ptx::tmem_ld32(t_half + 32, r1);
  ptx::tmem_ld_wait();
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float a0 = __uint_as_float(r0[2 * i]), a1 = __uint_as_float(r0[2 * i + 1]);
    float b0 = __uint_as_float(r1[2 * i]), b1 = __uint_as_float(r1[2 * i + 1]);
    if (kMasked) {
      a0 = (w0 >> (2 * i)) & 1u ? a0 : -INFINITY;
      a1 = (w0 >> (2 * i + 1)) & 1u ? a1 : -INFINITY;
      b0 = (w1 >> (2 * i)) & 1u ? b0 : -INFINITY;
      b1 = (w1 >> (2 * i + 1)) & 1u ? b1 : -INFINITY;
    }
    mx = ptx::max3(mx, a0, a1);
    mx = ptx::max3(mx, b0, b1);
  }
  smax_out = mx;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreadsTC, 2)
attn_fwd_tc_kernel(const AttnParams p,
                   const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v) {
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
  float* xch = reinterpret_cast<float*>(smem + L::off_xch);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = blockIdx.x;
  const int b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const int nk = p.Sk / p.BK;
  const int eps = kTileN / p.BK;        // list entries per step
  const int sps = p.BK / 32;            // 32-column sub-slots per entry

  int n_full = p.full_lens[b * p.fls[0] + h * p.fls[1] + static_cast<int64_t>(qblk) * p.fls[2]];  // line 107
  int n_part = p.part_lens[b * p.pls[0] + h * p.pls[1] + static_cast<int64_t>(qblk) * p.pls[2]];  // line 127
  n_full = min(max(n_full, 0), nk);
  n_part = min(max(n_part, 0), nk);
  const int total = n_full + n_part;
  const int n_steps = (total + eps - 1) / eps;
  const int n_plain = n_full / eps;     // leading steps made of full blocks only

  T* o_base = static_cast<T*>(p.o) + b * p.os[0] + h * p.os[1] + static_cast<int64_t>(qblk) * kTileM * p.os[2];

  if (total == 0) {                     // nothing attended: rows are 0, no tensor memory needed
    if (warp >= 2) {
      const int row = (warp & 3) * 32 + lane;
      uint4* dst = reinterpret_cast<uint4*>(o_base + static_cast<int64_t>(row) * p.os[2] + (D / 2) * ((warp - 2) >> 2));
#pragma unroll
      for (int i = 0; i < D / 16; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    return;
  }

  if (threadIdx.x == 0) {
    ptx::mbar_init(bar(BAR_Q), 1);
    ptx::mbar_init(bar(BAR_K_FULL), 1);
    ptx::mbar_init(bar(BAR_K_EMPTY), 1);
    ptx::mbar_init(bar(BAR_V_FULL), 1);
    ptx::mbar_init(bar(BAR_V_EMPTY), 1);
    ptx::mbar_init(bar(BAR_S_FULL), 1);
    ptx::mbar_init(bar(BAR_P_FULL), 256);
    ptx::mbar_init(bar(BAR_O_FULL), 1);
    ptx::mbar_init(bar(BAR_BITS_FULL0), 1);
    ptx::mbar_init(bar(BAR_BITS_FULL1), 1);
    ptx::mbar_init(bar(BAR_BITS_EMPTY0), 256);
    ptx::mbar_init(bar(BAR_BITS_EMPTY1), 256);
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
  const uint32_t tS = tmem_base;
  const uint32_t tO = tmem_base + 128;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      const int qb = p.qs[0] ? b : 0, qh = p.qs[1] ? h : 0;
      const int kb = p.ks[0] ? b : 0, kh = p.ks[1] ? h : 0;
      const int vb = p.vs[0] ? b : 0, vh = p.vs[1] ? h : 0;
      ptx::mbar_arrive_expect_tx(bar(BAR_Q), L::kTileBytes);
#pragma unroll
      for (int pnl = 0; pnl < D / 64; ++pnl)
        ptx::tma_load_4d(sQ + pnl * kPanelBytes, &tm_q, bar(BAR_Q), pnl * 64, qblk * kTileM, qh, qb);

      const int32_t* fids = p.full_ids + b * p.fis[0] + h * p.fis[1] + static_cast<int64_t>(qblk) * p.fis[2];
      const int32_t* pids = p.part_ids + b * p.pis[0] + h * p.pis[1] + static_cast<int64_t>(qblk) * p.pis[2];
      const uint32_t* bits_plane = p.bits + b * p.bits_sb + h * p.bits_sh;
      bool bad_index = false;
      auto entry_id = [&](int e) -> int {
        const int ee = e < total ? e : 0;         // slots past the end re-load the first listed block
        int id = ee < n_full ? fids[ee * p.fis[3]] : pids[(ee - n_full) * p.pis[3]];   // line 33
        if (static_cast<unsigned>(id) >= static_cast<unsigned>(nk)) { bad_index = true; id = 0; }
        return id;
      };
      int nxt[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) nxt[c] = (c < eps) ? entry_id(c) : 0;

      const uint32_t slot_bytes = static_cast<uint32_t>(p.BK) * 128u;
      bool ok = true;
      for (int j = 0; j < n_steps; ++j) {
        int cur[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) cur[c] = nxt[c];
        if (j + 1 < n_steps) {
#pragma unroll
          for (int c = 0; c < 4; ++c) nxt[c] = (c < eps) ? entry_id((j + 1) * eps + c) : 0;
        }
        // K tile: free once S(j-1) has been computed
        if (j > 0) ok = ptx::mbar_wait(bar(BAR_K_EMPTY), (j - 1) & 1, abort_flag);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bar(BAR_K_FULL), L::kTileBytes);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c < eps) {
#pragma unroll
            for (int pnl = 0; pnl < D / 64; ++pnl)
              ptx::tma_load_4d(sK + pnl * kPanelBytes + c * slot_bytes, &tm_k, bar(BAR_K_FULL),
                               pnl * 64, cur[c] * p.BK, kh, kb);
          }
        }
        // bit-mask tiles of the partial blocks of this step
        if (j >= n_plain) {
          const int u = j - n_plain, st = u & 1;
          if (u >= 2) ok = ptx::mbar_wait(bar(BAR_BITS_EMPTY0 + st), ((u >> 1) - 1) & 1, abort_flag);
          if (!ok) break;
          int n_tiles = 0;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int e = j * eps + c / sps;
            n_tiles += (e >= n_full && e < total) ? 1 : 0;
          }
          if (n_tiles > 0) ptx::mbar_arrive_expect_tx(bar(BAR_BITS_FULL0 + st), 512u * n_tiles);
          else ptx::mbar_arrive(bar(BAR_BITS_FULL0 + st));
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int ec = c / sps;
            const int e = j * eps + ec;
            if (e >= n_full && e < total) {
              const int64_t kb32 = static_cast<int64_t>(cur[ec]) * sps + (c % sps);
              const uint32_t* src = bits_plane + kb32 * p.Sq + qblk * kTileM;
              ptx::bulk_load(sBits + static_cast<uint32_t>(st * 4 + c) * 512u, src, 512u, bar(BAR_BITS_FULL0 + st));
            }
          }
        }
        // V tile: free once O += P.V (j-1) has been computed
        if (j > 0) ok = ptx::mbar_wait(bar(BAR_V_EMPTY), (j - 1) & 1, abort_flag);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bar(BAR_V_FULL), L::kTileBytes);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c < eps) {
#pragma unroll
            for (int pnl = 0; pnl < D / 64; ++pnl)
              ptx::tma_load_4d(sV + pnl * kPanelBytes + c * slot_bytes, &tm_v, bar(BAR_V_FULL),
                               pnl * 64, cur[c] * p.BK, vh, vb);
          }
        }
      }
      if (bad_index && p.dev_status != nullptr) atomicMax(p.dev_status, SA_DEV_BAD_INDEX);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = ptx::umma_idesc_f16(Fmt<T>::umma, kTileM, kTileN, 0);
      constexpr uint32_t idesc_o = ptx::umma_idesc_f16(Fmt<T>::umma, kTileM, D, 1);
      bool ok = ptx::mbar_wait(bar(BAR_Q), 0, abort_flag);
      for (int j = 0; j < n_steps && ok; ++j) {
        ok = ptx::mbar_wait(bar(BAR_K_FULL), j & 1, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {                      // S = Q.K^T  (line 40)
          const uint32_t off = (kk / 4) * kPanelBytes + (kk % 4) * 32u;
          ptx::mma_ss(tS, ptx::umma_desc_sw128(sQ + off, 16u), ptx::umma_desc_sw128(sK + off, 16u),
                      idesc_s, kk > 0 ? 1u : 0u);
        }
        ptx::mma_commit(bar(BAR_K_EMPTY));
        ptx::mma_commit(bar(BAR_S_FULL));
        ok = ptx::mbar_wait(bar(BAR_P_FULL), j & 1, abort_flag);
        if (!ok) break;
        ok = ptx::mbar_wait(bar(BAR_V_FULL), j & 1, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kTileN / 16; ++kk) {                 // O += P.V   (line 61)
          ptx::mma_ts(tO, tS + (kk / 4) * 64u + (kk % 4) * 8u, ptx::umma_desc_sw128(sV + kk * 2048u, kPanelBytes),
                      idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        ptx::mma_commit(bar(BAR_V_EMPTY));
        if (j == n_steps - 1) ptx::mma_commit(bar(BAR_O_FULL));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax
    // Thread = (query row, half of the 128 score columns).  Warps 2-5 take columns 0-63,
    // warps 6-9 columns 64-127; a warp may only touch the TMEM lanes of its quarter (warp % 4).
    const int lq = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = lq * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(lq * 32) << 16;
    const uint32_t tS_half = tS + lane_off + 64u * half;      // this half's scores; its P goes to the first 32 columns
    const uint32_t tO_half = tO + lane_off + (D / 2) * half;  // this half's share of the O columns
    const float scale = p.scale_log2;
    float m = -INFINITY, l = 0.f;                  // lines 103-104; l holds this half's partial sum
    bool ok = true;
    for (int j = 0; j < n_steps; ++j) {
      ok = ptx::mbar_wait(bar(BAR_S_FULL), j & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      const bool masked = j >= n_plain;
      uint32_t w0 = 0xffffffffu, w1 = 0xffffffffu;
      if (masked) {
        const int u = j - n_plain, st = u & 1;
        ok = ptx::mbar_wait(bar(BAR_BITS_FULL0 + st), (u >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int c0 = 2 * half, c1 = 2 * half + 1;
        const int e0 = j * eps + c0 / sps, e1 = j * eps + c1 / sps;
        w0 = e0 < n_full ? 0xffffffffu : (e0 < total ? bits_smem[(st * 4 + c0) * 128 + row] : 0u);
        w1 = e1 < n_full ? 0xffffffffu : (e1 < total ? bits_smem[(st * 4 + c1) * 128 + row] : 0u);
        ptx::mbar_arrive(bar(BAR_BITS_EMPTY0 + st));
      }
      float* xch_mine = xch + ((j & 1) * 2 + half) * 128 + row;
      const float* xch_other = xch + ((j & 1) * 2 + (half ^ 1)) * 128 + row;

      // Rows that already hold a finite running max exponentiate against it straight away
      // (one pass); the max only moves when a score exceeds it by more than the threshold.
      const bool slow = __any_sync(0xffffffffu, m == -INFINITY);
      float m_new = m, alpha = 1.f, m_ref = m;
      bool second_pass = true;
      if (!slow) {
        float sum, xmax;
        if (masked) softmax_pass<T, true>(tS_half, scale, m, w0, w1, sum, xmax);
        else        softmax_pass<T, false>(tS_half, scale, m, w0, w1, sum, xmax);
        *xch_mine = xmax;
        ptx::named_bar_sync(1 + lq, 64);
        const float xrow = fmaxf(xmax, *xch_other);
        if (!__any_sync(0xffffffffu, xrow > kRescaleThreshold)) {
          l += sum;
          second_pass = false;
        } else if (xrow > kRescaleThreshold) {
          m_new = m + xrow;
          alpha = ex2_approx(-xrow);                              // exp2(m - m_new), line 55
          m_ref = m_new;
        }
      } else {
        float smax;
        if (masked) max_pass<true>(tS_half, w0, w1, smax);
        else        max_pass<false>(tS_half, w0, w1, smax);
        *xch_mine = smax;
        ptx::named_bar_sync(1 + lq, 64);
        const float m_tile = fmaxf(smax, *xch_other) * scale;     // lines 48 / 50
        const float m_cand = fmaxf(m, m_tile);
        if (m == -INFINITY) { m_new = m_cand; }                   // nothing accumulated yet
        else if (m_cand > m + kRescaleThreshold) { m_new = m_cand; alpha = ex2_approx(m - m_new); }
        m_ref = (m_new == -INFINITY) ? 0.f : m_new;               // guard the reference lacks (line 53)
      }
      if (second_pass) {
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {     // acc *= alpha (line 58), this half's columns
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            uint32_t r[32];
            ptx::tmem_ld32(tO_half + c * 32, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            ptx::tmem_st32(tO_half + c * 32, r);
          }
        }
        float sum, xmax;
        if (masked) softmax_pass<T, true>(tS_half, scale, m_ref, w0, w1, sum, xmax);
        else        softmax_pass<T, false>(tS_half, scale, m_ref, w0, w1, sum, xmax);
        l = l * alpha + sum;                                      // line 57
        m = m_new;                                                // line 56
      }
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(BAR_P_FULL));
    }
    if (ok) {
      ok = ptx::mbar_wait(bar(BAR_O_FULL), 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      ptx::tc_fence_after();
      float* xch_mine = xch + ((n_steps & 1) * 2 + half) * 128 + row;
      const float* xch_other = xch + ((n_steps & 1) * 2 + (half ^ 1)) * 128 + row;
      *xch_mine = l;
      ptx::named_bar_sync(1 + lq, 64);
      const float l_row = l + *xch_other;
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;          // line 144, with 0 for an empty row
      uint4* dst = reinterpret_cast<uint4*>(o_base + static_cast<int64_t>(row) * p.os[2] + (D / 2) * half);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t r[32];
        ptx::tmem_ld32(tO_half + c * 32, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v;
          v.x = Fmt<T>::pack2(__uint_as_float(r[8 * i + 0]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
          v.y = Fmt<T>::pack2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
          v.z = Fmt<T>::pack2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
          v.w = Fmt<T>::pack2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
          dst[c * 4 + i] = v;                             // line 146
        }
      }
    }
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

bool tma_friendly(const void* base, const int64_t* st, int S) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return false;
  if (st[3] != 1) return false;
  if (st[2] <= 0 || st[2] % 8 != 0) return false;
  if (st[1] < 0 || st[1] % 8 != 0 || st[0] < 0 || st[0] % 8 != 0) return false;
  (void)S;
  return true;
}

template <typename T, int D>
int launch_inst(const AttnParams& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                cudaStream_t stream) {
  auto kernel = attn_fwd_tc_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(Smem<D>::dynamic_bytes));
  if (e != cudaSuccess) return SA_ERR_CUDA;
  dim3 grid(p.Sq / kTileM, p.B * p.H);
  kernel<<<grid, kThreadsTC, Smem<D>::dynamic_bytes, stream>>>(p, mq, mk, mv);
  return cudaGetLastError() == cudaSuccess ? SA_OK : SA_ERR_CUDA;
}

}  // namespace

int attn_tc_supported(const AttnParams& p) {
  if (p.dtype != SA_DTYPE_F16 && p.dtype != SA_DTYPE_BF16) return 0;
  if (p.D != 64 && p.D != 128) return 0;
  if (p.BQ != kTileM) return 0;
  if (p.BK != 32 && p.BK != 64 && p.BK != 128) return 0;
  if (p.Sq % kTileM != 0 || p.Sk % p.BK != 0) return 0;
  if (p.bits == nullptr) return 0;
  if (reinterpret_cast<uintptr_t>(p.bits) % 16 != 0 || p.bits_sb % 4 != 0 || p.bits_sh % 4 != 0) return 0;
  if (!(p.scale_log2 > 0.f) || !(p.scale_log2 < 1e30f)) return 0;
  if (!tma_friendly(p.q, p.qs, p.Sq) || !tma_friendly(p.k, p.ks, p.Sk) || !tma_friendly(p.v, p.vs, p.Sk)) return 0;
  if (reinterpret_cast<uintptr_t>(p.o) % 16 != 0 || p.os[3] != 1 || p.os[2] % 8 != 0 || p.os[1] % 8 != 0 ||
      p.os[0] % 8 != 0)
    return 0;
  return 1;
}

int launch_attn_tc(const AttnParams& p, cudaStream_t stream) {
  if (!attn_tc_supported(p)) return SA_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, p.q, p.dtype, p.B, p.H, p.Sq, p.D, p.qs, kTileM)) return SA_ERR_CUDA;
  if (!make_map(&mk, p.k, p.dtype, p.B, p.H, p.Sk, p.D, p.ks, p.BK)) return SA_ERR_CUDA;
  if (!make_map(&mv, p.v, p.dtype, p.B, p.H, p.Sk, p.D, p.vs, p.BK)) return SA_ERR_CUDA;
  if (p.dtype == SA_DTYPE_BF16) {
    return p.D == 128 ? launch_inst<__nv_bfloat16, 128>(p, mq, mk, mv, stream)
                      : launch_inst<__nv_bfloat16, 64>(p, mq, mk, mv, stream);
  }
  return p.D == 128 ? launch_inst<__half, 128>(p, mq, mk, mv, stream)
                    : launch_inst<__half, 64>(p, mq, mk, mv, stream);
}

}  // namespace sa
