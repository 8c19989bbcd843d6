// Backward pass of the block-sparse attention forward on the tensor cores (warp-level MMA, fp16 / bf16
// inputs, fp32 accumulation), head dims 64 and 128.
//
// The reference has no backward (README.md:61-65); the mathematics is that of attn_bwd_simt.cu:
//
//   P_ij  = exp(q_i.k_j * scale - lse_i)  on attended (i, j) of listed tiles, 0 elsewhere
//   D_i   = sum_d dO_id * O_id  (- the incoming gradient of lse_i, when there is one)
//   dV_j  = sum_i P_ij dO_i          dS_ij = P_ij * (dO_i.v_j - D_i)
//   dQ_i  = scale * sum_j dS_ij k_j  dK_j  = scale * sum_i dS_ij q_i
//
// One kernel template in two modes, no atomics (the result does not depend on the order CTAs run in):
//   mode 0 (dQ, also writes D): a CTA owns 32 query rows and walks the two kv-block lists of their
//     query block, the forward's walk;
//   mode 1 (dK, dV): a CTA owns 32 kv rows and walks the transposed (kv-major) lists of their kv block.
// In both the other side arrives in chunks of 32 rows staged in shared memory.  A warp owns 16 of the
// CTA's rows and needs nothing from the other warp: per chunk it forms two 16 x 32 products over the
// head dim (scores and dO.V^T; mma.sync m16n8k16, operands by ldmatrix), turns them into P and dS in
// its registers (rounded to the input type, as the forward rounds P before P.V: two adjacent 8-column
// accumulator tiles are one 16-column A operand), and accumulates 16 x D products over the chunk's 32
// rows.  The chunks are requested one ahead with cp.async (two buffers), the mask bytes of partial
// blocks with them.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "sa_common.cuh"

namespace sa {
namespace {

constexpr int kC = 32;            // rows of the other side per chunk
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// R = rows a CTA owns (32, 64 or 128: never more than the block size of its side, so that all of them
// walk the same lists); a warp owns 16 of them.
template <int D, int R> struct BwdSmem {
  static constexpr int kLd = D + 8;                                 // rows of the staged tiles (elements): 16 bytes of padding
  static constexpr size_t tile_a = static_cast<size_t>(R) * kLd * 2;          // bytes of one R x D tile
  static constexpr size_t tile_b = static_cast<size_t>(kC) * kLd * 2;         // bytes of one 32 x D tile
  static constexpr size_t off_a1 = 0, off_a2 = tile_a;
  static constexpr size_t off_b = 2 * tile_a;                                 // [2 buffers][2 tiles]
  static constexpr size_t off_mask = off_b + 4 * tile_b;                      // [2 buffers][R * 32] bytes
  static constexpr size_t off_stat = off_mask + 2 * static_cast<size_t>(R) * kC;             // own lse2[R], dsum[R]; chunk's [2][2][32]
  static constexpr size_t total = off_stat + (2 * R + 4 * kC) * 4;
};

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// four 8 x 8 matrices of 16-bit elements from shared memory; lane l gives the address of row l % 8 of
// matrix l / 8; register i of a lane holds elements (row lane / 4, columns 2 * (lane % 4) + {0, 1}) of
// matrix i -- of its transpose with kTrans
template <bool kTrans>
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
  if (kTrans)
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
  else
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// D (16 x 8, fp32) += A (16 x 16, row) . B (16 x 8, col).  With g = lane / 4, t = lane % 4:
// A: a0 (row g, k 2t..), a1 (row g+8, k 2t..), a2 (row g, k 2t+8..), a3 (row g+8, k 2t+8..);
// B: b0 (k 2t.., n g), b1 (k 2t+8.., n g);  D: d0 d1 (row g, n 2t 2t+1), d2 d3 (row g+8, n 2t 2t+1).
template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// `rows` rows x D elements from global memory (unit stride along D, 16-byte aligned rows) into a padded
// tile, asynchronously (cp.async, 16 bytes each)
template <typename T, int D, int kThreads>
__device__ __forceinline__ void load_tile_async(T* dst, const T* src, int64_t row_stride, int rows, int tid) {
  constexpr int kLd = D + 8;
  constexpr int kVecPerRow = D / 8;                       // 16-byte vectors
  for (int e = tid; e < rows * kVecPerRow; e += kThreads) {
    const int r = e / kVecPerRow, c = e % kVecPerRow;
    cp_async_16(dst + r * kLd + c * 8, src + static_cast<int64_t>(r) * row_stride + c * 8);
  }
}

template <typename T, int D, int R, int MODE>
__global__ void __launch_bounds__(2 * R)
attn_bwd_mma_kernel(const AttnBwdParams p, const int mask_vec) {
  using S = BwdSmem<D, R>;
  constexpr int kLd = S::kLd;
  constexpr int kThreads = 2 * R;
  extern __shared__ __align__(128) uint8_t smem[];
  T* sA1 = reinterpret_cast<T*>(smem + S::off_a1);
  T* sA2 = reinterpret_cast<T*>(smem + S::off_a2);
  T* sB = reinterpret_cast<T*>(smem + S::off_b);                       // buffer u & 1: tiles B1 then B2
  uint8_t* s_mask = smem + S::off_mask;                                // buffer u & 1: the chunk's mask bytes
  float* s_lse2 = reinterpret_cast<float*>(smem + S::off_stat);      // own rows (mode 0)
  float* s_dsum = s_lse2 + R;
  float* c_stat = s_lse2 + 2 * R;                                      // the chunk's query rows (mode 1): [buffer][lse2 | dsum][32]
  const AttnParams& f = p.fwd;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int rows_total = MODE == 0 ? f.Sq : f.Sk;
  const int groups = rows_total / R;
  const int row0 = static_cast<int>(blockIdx.x % groups) * R;         // first row this CTA owns
  const int bh = static_cast<int>(blockIdx.x / groups);
  const int b = bh / f.H, h = bh % f.H;
  const int own_blk = row0 / (MODE == 0 ? f.BQ : f.BK);
  const int n_other = MODE == 0 ? f.Sk / f.BK : f.Sq / f.BQ;          // blocks on the other side
  const int other_rows = MODE == 0 ? f.BK : f.BQ;
  const int cpb = other_rows / kC;                                    // chunks per block of the other side

  const T* qbase = static_cast<const T*>(f.q) + b * f.qs[0] + h * f.qs[1];
  const T* kbase = static_cast<const T*>(f.k) + b * f.ks[0] + h * f.ks[1];
  const T* vbase = static_cast<const T*>(f.v) + b * f.vs[0] + h * f.vs[1];
  const T* gbase = static_cast<const T*>(p.d_o) + b * p.dos[0] + h * p.dos[1];
  const uint8_t* mbase = f.mask + b * f.ms[0] + h * f.ms[1];
  const int64_t stat0 = (static_cast<int64_t>(b) * f.H + h) * f.Sq;

  // the two lists this CTA walks: the full one first, then the partial one (the forward's order)
  const int32_t *fids, *pids;
  int64_t fstr, pstr;
  int nf, np;
  if (MODE == 0) {
    fids = f.full_ids + b * f.fis[0] + h * f.fis[1] + static_cast<int64_t>(own_blk) * f.fis[2];
    pids = f.part_ids + b * f.pis[0] + h * f.pis[1] + static_cast<int64_t>(own_blk) * f.pis[2];
    fstr = f.fis[3]; pstr = f.pis[3];
    nf = f.full_lens[b * f.fls[0] + h * f.fls[1] + static_cast<int64_t>(own_blk) * f.fls[2]];
    np = f.part_lens[b * f.pls[0] + h * f.pls[1] + static_cast<int64_t>(own_blk) * f.pls[2]];
  } else {
    fids = p.t_full_ids + b * p.tfis[0] + h * p.tfis[1] + static_cast<int64_t>(own_blk) * p.tfis[2];
    pids = p.t_part_ids + b * p.tpis[0] + h * p.tpis[1] + static_cast<int64_t>(own_blk) * p.tpis[2];
    fstr = p.tfis[3]; pstr = p.tpis[3];
    nf = p.t_full_lens[b * p.tfls[0] + h * p.tfls[1] + static_cast<int64_t>(own_blk) * p.tfls[2]];
    np = p.t_part_lens[b * p.tpls[0] + h * p.tpls[1] + static_cast<int64_t>(own_blk) * p.tpls[2]];
  }
  nf = min(max(nf, 0), n_other);
  np = min(max(np, 0), n_other);
  const int total_chunks = (nf + np) * cpb;

  // chunk u of the walk: first row on the other side (-1 for an id out of range), and whether the mask applies
  auto chunk_of = [&](int u, bool& masked) -> int {
    const int e = u / cpb, sub = (u - e * cpb) * kC;
    masked = e >= nf;
    const int id = masked ? pids[(e - nf) * pstr] : fids[e * fstr];
    if (id < 0 || id >= n_other) return -1;
    return id * other_rows + sub;
  };
  // requests chunk u into buffer u & 1 (every thread takes part; one cp.async group per chunk)
  auto request = [&](int u) {
    bool masked;
    const int c0 = chunk_of(u, masked);
    const int buf = u & 1;
    if (c0 >= 0) {
      T* b1 = sB + static_cast<size_t>(buf) * 2 * kC * kLd;
      T* b2 = b1 + kC * kLd;
      if (MODE == 0) {
        load_tile_async<T, D, kThreads>(b1, kbase + static_cast<int64_t>(c0) * f.ks[2], f.ks[2], kC, tid);
        load_tile_async<T, D, kThreads>(b2, vbase + static_cast<int64_t>(c0) * f.vs[2], f.vs[2], kC, tid);
      } else {
        load_tile_async<T, D, kThreads>(b1, qbase + static_cast<int64_t>(c0) * f.qs[2], f.qs[2], kC, tid);
        load_tile_async<T, D, kThreads>(b2, gbase + static_cast<int64_t>(c0) * p.dos[2], p.dos[2], kC, tid);
        if (tid < kC) {
          c_stat[buf * 2 * kC + tid] = f.lse[stat0 + c0 + tid] * kLog2e;
          c_stat[buf * 2 * kC + kC + tid] = p.dsum[stat0 + c0 + tid];
        }
      }
      if (masked && mask_vec) {
        // the chunk's mask bytes, [query row][kv row]: R x 32 (mode 0) or 32 x R (mode 1)
        constexpr int kQ = MODE == 0 ? R : kC, kK = MODE == 0 ? kC : R;
        const int q0 = MODE == 0 ? row0 : c0, k0 = MODE == 0 ? c0 : row0;
        uint8_t* dstm = s_mask + static_cast<size_t>(buf) * R * kC;
        for (int e = tid; e < kQ * (kK / 16); e += kThreads) {
          const int qr = e / (kK / 16), piece = e % (kK / 16);
          cp_async_16(dstm + qr * kK + piece * 16, mbase + static_cast<int64_t>(q0 + qr) * f.ms[2] + k0 + piece * 16);
        }
      }
    }
    cp_async_commit();
  };

  // the CTA's own rows: Q and dO (mode 0), K and V (mode 1)
  if (MODE == 0) {
    load_tile_async<T, D, kThreads>(sA1, qbase + static_cast<int64_t>(row0) * f.qs[2], f.qs[2], R, tid);
    load_tile_async<T, D, kThreads>(sA2, gbase + static_cast<int64_t>(row0) * p.dos[2], p.dos[2], R, tid);
    // D_i = sum_d dO_id O_id (- d_lse_i): two threads per row
    const int r = tid >> 1, half = tid & 1;
    const T* o = static_cast<const T*>(f.o) + b * f.os[0] + h * f.os[1] + static_cast<int64_t>(row0 + r) * f.os[2];
    const T* g = gbase + static_cast<int64_t>(row0 + r) * p.dos[2];
    float acc = 0.f;
    for (int d = half * (D / 2); d < (half + 1) * (D / 2); d += 8) {
      const uint4 ov = *reinterpret_cast<const uint4*>(o + d), gv = *reinterpret_cast<const uint4*>(g + d);
      const T* oe = reinterpret_cast<const T*>(&ov);
      const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf(to_float<T>(ge[i]), to_float<T>(oe[i]), acc);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    if (half == 0) {
      const int64_t stat = stat0 + row0 + r;
      if (p.d_lse != nullptr) acc -= p.d_lse[stat];
      p.dsum[stat] = acc;
      s_dsum[r] = acc;
      s_lse2[r] = f.lse[stat] * kLog2e;              // -inf for a row with no attended key: no gradient
    }
  } else {
    load_tile_async<T, D, kThreads>(sA1, kbase + static_cast<int64_t>(row0) * f.ks[2], f.ks[2], R, tid);
    load_tile_async<T, D, kThreads>(sA2, vbase + static_cast<int64_t>(row0) * f.vs[2], f.vs[2], R, tid);
  }
  cp_async_commit();

  // Accumulators of this warp's 16 rows, as 16 x 8 tiles of the MMA: dQ (mode 0); dV and dK (mode 1).
  constexpr int kDT = D / 8;
  float acc1[kDT][4];
  float acc2[MODE == 1 ? kDT : 1][4];
#pragma unroll
  for (int n = 0; n < kDT; ++n) { acc1[n][0] = acc1[n][1] = acc1[n][2] = acc1[n][3] = 0.f; }
  if constexpr (MODE == 1) {
#pragma unroll
    for (int n = 0; n < kDT; ++n) { acc2[n][0] = acc2[n][1] = acc2[n][2] = acc2[n][3] = 0.f; }
  }

  const int g = lane >> 2, t4 = lane & 3;
  // ldmatrix addresses: A operand (this warp's rows, k along the head dim): row lane % 16, +8 columns for lanes >= 16
  const T* a1_ld = sA1 + (warp * 16 + (lane & 15)) * kLd + (lane >> 4) * 8;
  const T* a2_ld = sA2 + (warp * 16 + (lane & 15)) * kLd + (lane >> 4) * 8;
  // B operand of the first products, B(k, n) = tile[n][k] (no transpose): matrices (n 0-7, k 0-7), (n 0-7, k 8-15),
  // (n 8-15, k 0-7), (n 8-15, k 8-15)
  const int bt_row = ((lane >> 4) << 3) + (lane & 7), bt_col = ((lane >> 3) & 1) * 8;
  // B operand of the accumulating products, B(k, n) = tile[k][n] (transposed load): matrices (k 0-7, n 0-7),
  // (k 8-15, n 0-7), (k 0-7, n 8-15), (k 8-15, n 8-15)
  const int bn_row = (((lane >> 3) & 1) << 3) + (lane & 7), bn_col = (lane >> 4) * 8;
  float own_lse2[2] = {0.f, 0.f}, own_dsum[2] = {0.f, 0.f};

  if (total_chunks > 0) request(0);
#pragma unroll 1
  for (int u = 0; u < total_chunks; ++u) {
    // One barrier per chunk: behind it chunk u has landed for every thread, and every warp is done with
    // chunk u-1, whose buffer the next chunk is then requested into (it travels while this one is worked on).
    cp_async_wait<0>();
    __syncthreads();
    if (u + 1 < total_chunks) request(u + 1);
    if (MODE == 0 && u == 0) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        own_lse2[hh] = s_lse2[warp * 16 + g + 8 * hh];
        own_dsum[hh] = s_dsum[warp * 16 + g + 8 * hh];
      }
    }
    bool masked;
    const int c0 = chunk_of(u, masked);
    const int buf = u & 1;
    if (c0 < 0) {
      if (tid == 0 && f.dev_status != nullptr) atomicMax(f.dev_status, SA_DEV_BAD_INDEX);
    } else {
      const T* sB1 = sB + static_cast<size_t>(buf) * 2 * kC * kLd;
      const T* sB2 = sB1 + kC * kLd;
      // T1 = A1_w . B1^T (scores) and T2 = A2_w . B2^T (16 x 32 each, over the head dim), in registers
      float t1[kC / 8][4], t2[kC / 8][4];
#pragma unroll
      for (int n = 0; n < kC / 8; ++n) {
        t1[n][0] = t1[n][1] = t1[n][2] = t1[n][3] = 0.f;
        t2[n][0] = t2[n][1] = t2[n][2] = t2[n][3] = 0.f;
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a1[4], a2[4];
        ldmatrix_x4<false>(a1, a1_ld + kk * 16);
        ldmatrix_x4<false>(a2, a2_ld + kk * 16);
#pragma unroll
        for (int np = 0; np < kC / 16; ++np) {          // pairs of 8-column tiles
          uint32_t b1[4], b2[4];
          ldmatrix_x4<false>(b1, sB1 + (np * 16 + bt_row) * kLd + kk * 16 + bt_col);
          ldmatrix_x4<false>(b2, sB2 + (np * 16 + bt_row) * kLd + kk * 16 + bt_col);
          mma_16816<T>(t1[2 * np], a1, b1[0], b1[1]);
          mma_16816<T>(t1[2 * np + 1], a1, b1[2], b1[3]);
          mma_16816<T>(t2[2 * np], a2, b2[0], b2[1]);
          mma_16816<T>(t2[2 * np + 1], a2, b2[2], b2[3]);
        }
      }

      // P and dS in place: element (row g + 8 * (i / 2), column 8 * n + 2 * t4 + (i & 1)) of the chunk
      const uint8_t* sm = s_mask + static_cast<size_t>(buf) * R * kC;
      const float* cs = c_stat + buf * 2 * kC;
#pragma unroll
      for (int n = 0; n < kC / 8; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = warp * 16 + g + 8 * (i >> 1);    // row of the CTA
          const int col = 8 * n + 2 * t4 + (i & 1);      // column of the chunk
          float lse2, dsum;
          if (MODE == 0) { lse2 = own_lse2[i >> 1]; dsum = own_dsum[i >> 1]; }
          else           { lse2 = cs[col]; dsum = cs[kC + col]; }
          bool attend = lse2 > -INFINITY;
          if (masked && attend) {
            if (mask_vec) {
              attend = (MODE == 0 ? sm[r * kC + col] : sm[col * R + r]) != 0;
            } else {
              const int qrow = MODE == 0 ? row0 + r : c0 + col, krow = MODE == 0 ? c0 + col : row0 + r;
              attend = mbase[static_cast<int64_t>(qrow) * f.ms[2] + static_cast<int64_t>(krow) * f.ms[3]] != 0;
            }
          }
          const float pe = attend ? exp2f(t1[n][i] * f.scale_log2 - lse2) : 0.f;
          t1[n][i] = pe;
          t2[n][i] = pe * (t2[n][i] - dsum);
        }
      }

      // mode 0: dQ_w += dS . K_chunk; mode 1: dV_w += P . dO_chunk, dK_w += dS . Q_chunk.  Two adjacent 8-column
      // tiles of the first products are one 16-column A operand of these (rounded to the input type).
#pragma unroll
      for (int ks = 0; ks < kC / 16; ++ks) {
        uint32_t e_p[4], e_ds[4];
        e_ds[0] = pack_pair<T>(t2[2 * ks][0], t2[2 * ks][1]);
        e_ds[1] = pack_pair<T>(t2[2 * ks][2], t2[2 * ks][3]);
        e_ds[2] = pack_pair<T>(t2[2 * ks + 1][0], t2[2 * ks + 1][1]);
        e_ds[3] = pack_pair<T>(t2[2 * ks + 1][2], t2[2 * ks + 1][3]);
        if (MODE == 1) {
          e_p[0] = pack_pair<T>(t1[2 * ks][0], t1[2 * ks][1]);
          e_p[1] = pack_pair<T>(t1[2 * ks][2], t1[2 * ks][3]);
          e_p[2] = pack_pair<T>(t1[2 * ks + 1][0], t1[2 * ks + 1][1]);
          e_p[3] = pack_pair<T>(t1[2 * ks + 1][2], t1[2 * ks + 1][3]);
        }
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {           // pairs of 8-column tiles of the head dim
          uint32_t b1[4];
          ldmatrix_x4<true>(b1, sB1 + (ks * 16 + bn_row) * kLd + dp * 16 + bn_col);
          if constexpr (MODE == 0) {
            mma_16816<T>(acc1[2 * dp], e_ds, b1[0], b1[1]);
            mma_16816<T>(acc1[2 * dp + 1], e_ds, b1[2], b1[3]);
          } else {
            uint32_t b2[4];
            ldmatrix_x4<true>(b2, sB2 + (ks * 16 + bn_row) * kLd + dp * 16 + bn_col);
            mma_16816<T>(acc1[2 * dp], e_p, b2[0], b2[1]);          // dV
            mma_16816<T>(acc1[2 * dp + 1], e_p, b2[2], b2[3]);
            mma_16816<T>(acc2[2 * dp], e_ds, b1[0], b1[1]);         // dK
            mma_16816<T>(acc2[2 * dp + 1], e_ds, b1[2], b1[3]);
          }
        }
      }
    }
  }
  cp_async_wait<0>();

  // write the warp's 16 rows out: a lane holds columns 8 * n + 2 * t4 + {0, 1} of rows g and g + 8
  const float scale = f.scale_log2 * kLn2;
  auto write_out = [&](float (*acc)[4], T* out_base, int64_t row_stride, float factor) {
#pragma unroll
    for (int n = 0; n < kDT; ++n) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        T* dst = out_base + static_cast<int64_t>(warp * 16 + g + 8 * hh) * row_stride + 8 * n + 2 * t4;
        *reinterpret_cast<uint32_t*>(dst) = pack_pair<T>(acc[n][2 * hh] * factor, acc[n][2 * hh + 1] * factor);
      }
    }
  };
  if constexpr (MODE == 0) {
    T* dq = static_cast<T*>(p.dq) + b * p.dqs[0] + h * p.dqs[1] + static_cast<int64_t>(row0) * p.dqs[2];
    write_out(acc1, dq, p.dqs[2], scale);
  } else {
    T* dv = static_cast<T*>(p.dv) + b * p.dvs[0] + h * p.dvs[1] + static_cast<int64_t>(row0) * p.dvs[2];
    T* dk = static_cast<T*>(p.dk) + b * p.dks[0] + h * p.dks[1] + static_cast<int64_t>(row0) * p.dks[2];
    write_out(acc1, dv, p.dvs[2], 1.f);
    write_out(acc2, dk, p.dks[2], scale);
  }
}

bool vec_ok(const void* base, const int64_t* st) {
  return reinterpret_cast<uintptr_t>(base) % 16 == 0 && st[3] == 1 && st[2] % 8 == 0 && st[1] % 8 == 0 && st[0] % 8 == 0;
}

template <typename T, int D, int R, int MODE>
cudaError_t launch_one(const AttnBwdParams& p, int mask_vec, cudaStream_t stream) {
  const AttnParams& f = p.fwd;
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return cudaErrorNoDevice;
  auto kernel = attn_bwd_mma_kernel<T, D, R, MODE>;
  constexpr size_t smem = BwdSmem<D, R>::total;
  static std::once_flag once[kMaxDevices];
  static cudaError_t attr[kMaxDevices];
  std::call_once(once[info->ordinal], [&] {
    attr[info->ordinal] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  });
  if (attr[info->ordinal] != cudaSuccess) return attr[info->ordinal];
  const long long ctas = static_cast<long long>((MODE == 0 ? f.Sq : f.Sk) / R) * f.B * f.H;
  if (ctas <= 0 || ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  kernel<<<static_cast<unsigned>(ctas), 2 * R, smem, stream>>>(p, mask_vec);
  return cudaGetLastError();
}

// rows per CTA: the largest of 128 / 64 / 32 that divides the block size of the CTA's side
template <typename T, int D, int MODE>
cudaError_t launch_mode(const AttnBwdParams& p, int mask_vec, cudaStream_t stream) {
  const int blk = MODE == 0 ? p.fwd.BQ : p.fwd.BK;
  if (blk % 64 == 0) return launch_one<T, D, 64, MODE>(p, mask_vec, stream);
  return launch_one<T, D, 32, MODE>(p, mask_vec, stream);
}

template <typename T, int D>
cudaError_t launch_both(const AttnBwdParams& p, cudaStream_t stream) {
  const AttnParams& f = p.fwd;
  // the mask chunks are staged with 16-byte copies when its rows allow it
  const int mask_vec = reinterpret_cast<uintptr_t>(f.mask) % 16 == 0 && f.ms[3] == 1 && f.ms[2] % 16 == 0 &&
                       f.ms[1] % 16 == 0 && f.ms[0] % 16 == 0;
  cudaError_t e = launch_mode<T, D, 0>(p, mask_vec, stream);
  if (e != cudaSuccess) return e;
  return launch_mode<T, D, 1>(p, mask_vec, stream);           // reads D from the first
}

}  // namespace

int attn_bwd_mma_supported(const AttnBwdParams& p) {
  const AttnParams& f = p.fwd;
  if (f.dtype != SA_DTYPE_F16 && f.dtype != SA_DTYPE_BF16) return 0;
  if (f.D != 64 && f.D != 128) return 0;
  if (f.BQ % 32 != 0 || f.BK % 32 != 0 || f.Sq % f.BQ != 0 || f.Sk % f.BK != 0) return 0;
  return vec_ok(f.q, f.qs) && vec_ok(f.k, f.ks) && vec_ok(f.v, f.vs) && vec_ok(f.o, f.os) && vec_ok(p.d_o, p.dos) &&
         vec_ok(p.dq, p.dqs) && vec_ok(p.dk, p.dks) && vec_ok(p.dv, p.dvs);
}

cudaError_t launch_attn_bwd_mma(const AttnBwdParams& p, cudaStream_t stream) {
  const AttnParams& f = p.fwd;
  if (f.dtype == SA_DTYPE_BF16)
    return f.D == 128 ? launch_both<__nv_bfloat16, 128>(p, stream) : launch_both<__nv_bfloat16, 64>(p, stream);
  return f.D == 128 ? launch_both<__half, 128>(p, stream) : launch_both<__half, 64>(p, stream);
}

}  // namespace sa
