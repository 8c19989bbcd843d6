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
// head dim (scores and dO.V^T), turns them into P and dS element by element through shared memory
// (rounded to the input type, as the forward rounds P before P.V), and accumulates 16 x D products
// over the chunk's 32 rows.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <mma.h>

#include <mutex>

#include "sa_common.cuh"

namespace sa {
namespace {

using namespace nvcuda;

constexpr int kR = 32;            // rows a CTA owns
constexpr int kC = 32;            // rows of the other side per chunk
constexpr int kWarps = kR / 16;
constexpr int kThreadsMma = 32 * kWarps;
constexpr int kLdT = kC + 4;      // fp32 scratch rows (floats)
constexpr int kLdE = kC + 8;      // P / dS rows (elements)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int D> struct BwdSmem {
  static constexpr int kLd = D + 8;                                 // rows of the staged tiles (elements): 16 bytes of padding
  static constexpr size_t tile = static_cast<size_t>(kR) * kLd * 2;           // bytes of one 32 x D tile
  static constexpr size_t off_a1 = 0, off_a2 = tile, off_b1 = 2 * tile, off_b2 = 3 * tile;
  static constexpr size_t off_t = 4 * tile;                                   // [warp][2][16][kLdT] float
  static constexpr size_t off_e = off_t + static_cast<size_t>(kWarps) * 2 * 16 * kLdT * 4;   // [warp][2][16][kLdE] T
  static constexpr size_t off_stat = off_e + static_cast<size_t>(kWarps) * 2 * 16 * kLdE * 2;  // lse2[32], dsum[32] (own rows), then the chunk's
  static constexpr size_t total = off_stat + 4 * 32 * 4;
};

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

// 32 rows x D elements from global memory (unit stride along D, 16-byte aligned rows) into a padded tile
template <typename T, int D>
__device__ __forceinline__ void load_tile(T* dst, const T* src, int64_t row_stride, int tid) {
  constexpr int kLd = BwdSmem<D>::kLd;
  constexpr int kVecPerRow = D / 8;                       // 16-byte vectors
  for (int e = tid; e < kR * kVecPerRow; e += kThreadsMma) {
    const int r = e / kVecPerRow, c = e % kVecPerRow;
    const uint4 v = *reinterpret_cast<const uint4*>(src + static_cast<int64_t>(r) * row_stride + c * 8);
    *reinterpret_cast<uint4*>(dst + r * kLd + c * 8) = v;
  }
}

template <typename T, int D, int MODE>
__global__ void __launch_bounds__(kThreadsMma)
attn_bwd_mma_kernel(const AttnBwdParams p) {
  using S = BwdSmem<D>;
  constexpr int kLd = S::kLd;
  extern __shared__ __align__(128) uint8_t smem[];
  T* sA1 = reinterpret_cast<T*>(smem + S::off_a1);
  T* sA2 = reinterpret_cast<T*>(smem + S::off_a2);
  T* sB1 = reinterpret_cast<T*>(smem + S::off_b1);
  T* sB2 = reinterpret_cast<T*>(smem + S::off_b2);
  float* s_lse2 = reinterpret_cast<float*>(smem + S::off_stat);      // own rows (mode 0) / unused (mode 1)
  float* s_dsum = s_lse2 + 32;
  float* c_lse2 = s_lse2 + 64;                                        // the chunk's query rows (mode 1)
  float* c_dsum = s_lse2 + 96;
  const AttnParams& f = p.fwd;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* sT = reinterpret_cast<float*>(smem + S::off_t) + warp * 2 * 16 * kLdT;
  T* sE = reinterpret_cast<T*>(smem + S::off_e) + warp * 2 * 16 * kLdE;

  const int rows_total = MODE == 0 ? f.Sq : f.Sk;
  const int groups = rows_total / kR;
  const int row0 = static_cast<int>(blockIdx.x % groups) * kR;        // first row this CTA owns
  const int bh = static_cast<int>(blockIdx.x / groups);
  const int b = bh / f.H, h = bh % f.H;
  const int own_blk = row0 / (MODE == 0 ? f.BQ : f.BK);
  const int n_other = MODE == 0 ? f.Sk / f.BK : f.Sq / f.BQ;          // blocks on the other side
  const int other_rows = MODE == 0 ? f.BK : f.BQ;

  const T* qbase = static_cast<const T*>(f.q) + b * f.qs[0] + h * f.qs[1];
  const T* kbase = static_cast<const T*>(f.k) + b * f.ks[0] + h * f.ks[1];
  const T* vbase = static_cast<const T*>(f.v) + b * f.vs[0] + h * f.vs[1];
  const T* gbase = static_cast<const T*>(p.d_o) + b * p.dos[0] + h * p.dos[1];
  const uint8_t* mbase = f.mask + b * f.ms[0] + h * f.ms[1];
  const int64_t stat0 = (static_cast<int64_t>(b) * f.H + h) * f.Sq;

  // the CTA's own rows: Q and dO (mode 0), K and V (mode 1)
  if (MODE == 0) {
    load_tile<T, D>(sA1, qbase + static_cast<int64_t>(row0) * f.qs[2], f.qs[2], tid);
    load_tile<T, D>(sA2, gbase + static_cast<int64_t>(row0) * p.dos[2], p.dos[2], tid);
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
    load_tile<T, D>(sA1, kbase + static_cast<int64_t>(row0) * f.ks[2], f.ks[2], tid);
    load_tile<T, D>(sA2, vbase + static_cast<int64_t>(row0) * f.vs[2], f.vs[2], tid);
  }

  // accumulators of this warp's 16 rows: dQ (mode 0); dV and dK (mode 1)
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc1[D / 16];
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc2[MODE == 1 ? D / 16 : 1];
#pragma unroll
  for (int n = 0; n < D / 16; ++n) wmma::fill_fragment(acc1[n], 0.f);
  if constexpr (MODE == 1) {
#pragma unroll
    for (int n = 0; n < D / 16; ++n) wmma::fill_fragment(acc2[n], 0.f);
  }

  const T* a1_w = sA1 + warp * 16 * kLd;
  const T* a2_w = sA2 + warp * 16 * kLd;

#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const bool masked = pass == 1;
    const int32_t* ids;
    int64_t id_stride;
    int n_given;
    if (MODE == 0) {
      ids = masked ? f.part_ids + b * f.pis[0] + h * f.pis[1] + static_cast<int64_t>(own_blk) * f.pis[2]
                   : f.full_ids + b * f.fis[0] + h * f.fis[1] + static_cast<int64_t>(own_blk) * f.fis[2];
      id_stride = masked ? f.pis[3] : f.fis[3];
      n_given = masked ? f.part_lens[b * f.pls[0] + h * f.pls[1] + static_cast<int64_t>(own_blk) * f.pls[2]]
                       : f.full_lens[b * f.fls[0] + h * f.fls[1] + static_cast<int64_t>(own_blk) * f.fls[2]];
    } else {
      ids = masked ? p.t_part_ids + b * p.tpis[0] + h * p.tpis[1] + static_cast<int64_t>(own_blk) * p.tpis[2]
                   : p.t_full_ids + b * p.tfis[0] + h * p.tfis[1] + static_cast<int64_t>(own_blk) * p.tfis[2];
      id_stride = masked ? p.tpis[3] : p.tfis[3];
      n_given = masked ? p.t_part_lens[b * p.tpls[0] + h * p.tpls[1] + static_cast<int64_t>(own_blk) * p.tpls[2]]
                       : p.t_full_lens[b * p.tfls[0] + h * p.tfls[1] + static_cast<int64_t>(own_blk) * p.tfls[2]];
    }
    const int n = min(max(n_given, 0), n_other);
#pragma unroll 1
    for (int t = 0; t < n; ++t) {
      const int id = ids[t * id_stride];
      if (id < 0 || id >= n_other) {
        if (tid == 0 && f.dev_status != nullptr) atomicMax(f.dev_status, SA_DEV_BAD_INDEX);
        continue;
      }
#pragma unroll 1
      for (int sub = 0; sub < other_rows; sub += kC) {
        const int c0 = id * other_rows + sub;           // first row of the chunk on the other side
        __syncthreads();                                // every warp is done with the previous chunk's tiles
        if (MODE == 0) {
          load_tile<T, D>(sB1, kbase + static_cast<int64_t>(c0) * f.ks[2], f.ks[2], tid);
          load_tile<T, D>(sB2, vbase + static_cast<int64_t>(c0) * f.vs[2], f.vs[2], tid);
        } else {
          load_tile<T, D>(sB1, qbase + static_cast<int64_t>(c0) * f.qs[2], f.qs[2], tid);
          load_tile<T, D>(sB2, gbase + static_cast<int64_t>(c0) * p.dos[2], p.dos[2], tid);
          if (tid < kC) {
            c_lse2[tid] = f.lse[stat0 + c0 + tid] * kLog2e;
            c_dsum[tid] = p.dsum[stat0 + c0 + tid];
          }
        }
        __syncthreads();

        // T1 = A1_w . B1^T and T2 = A2_w . B2^T (16 x 32 each, over the head dim) into this warp's scratch
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const T* a_w = which == 0 ? a1_w : a2_w;
          const T* bt = which == 0 ? sB1 : sB2;
#pragma unroll
          for (int nf = 0; nf < kC / 16; ++nf) {
            wmma::fragment<wmma::accumulator, 16, 16, 16, float> c;
            wmma::fill_fragment(c, 0.f);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::row_major> a;
              wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::col_major> bm;
              wmma::load_matrix_sync(a, a_w + kk * 16, kLd);
              wmma::load_matrix_sync(bm, bt + nf * 16 * kLd + kk * 16, kLd);     // (k, n) = B[n][k]
              wmma::mma_sync(c, a, bm, c);
            }
            wmma::store_matrix_sync(sT + which * 16 * kLdT + nf * 16, c, kLdT, wmma::mem_row_major);
          }
        }
        __syncwarp();

        // P and dS, element by element: lane = column of the chunk, 16 rows each
        {
          const int col = lane;
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int r = warp * 16 + i;                 // row of the CTA
            const float t1 = sT[i * kLdT + col], t2 = sT[16 * kLdT + i * kLdT + col];
            float lse2, dsum;
            int qrow, krow;
            if (MODE == 0) { lse2 = s_lse2[r]; dsum = s_dsum[r]; qrow = row0 + r; krow = c0 + col; }
            else           { lse2 = c_lse2[col]; dsum = c_dsum[col]; qrow = c0 + col; krow = row0 + r; }
            bool attend = lse2 > -INFINITY;
            if (masked && attend)
              attend = mbase[static_cast<int64_t>(qrow) * f.ms[2] + static_cast<int64_t>(krow) * f.ms[3]] != 0;
            const float pe = attend ? exp2f(t1 * f.scale_log2 - lse2) : 0.f;
            const float ds = pe * (t2 - dsum);
            sE[i * kLdE + col] = from_float<T>(pe);
            sE[16 * kLdE + i * kLdE + col] = from_float<T>(ds);
          }
        }
        __syncwarp();

        // mode 0: dQ_w += dS . K_chunk; mode 1: dV_w += P^T-rows . dO_chunk, dK_w += dS . Q_chunk
#pragma unroll
        for (int kk = 0; kk < kC / 16; ++kk) {
          wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::row_major> e_p, e_ds;
          wmma::load_matrix_sync(e_ds, sE + 16 * kLdE + kk * 16, kLdE);
          if (MODE == 1) wmma::load_matrix_sync(e_p, sE + kk * 16, kLdE);
#pragma unroll
          for (int nf = 0; nf < D / 16; ++nf) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::row_major> b1;
            wmma::load_matrix_sync(b1, sB1 + kk * 16 * kLd + nf * 16, kLd);
            if constexpr (MODE == 0) {
              wmma::mma_sync(acc1[nf], e_ds, b1, acc1[nf]);
            } else {
              wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::row_major> b2;
              wmma::load_matrix_sync(b2, sB2 + kk * 16 * kLd + nf * 16, kLd);
              wmma::mma_sync(acc1[nf], e_p, b2, acc1[nf]);        // dV
              wmma::mma_sync(acc2[nf], e_ds, b1, acc2[nf]);       // dK
            }
          }
        }
      }
    }
  }

  // write the warp's 16 rows out, 16 columns at a time, through its scratch
  const float scale = f.scale_log2 * kLn2;
  __syncwarp();
  auto write_out = [&](wmma::fragment<wmma::accumulator, 16, 16, 16, float>* acc, T* out_base, int64_t row_stride,
                       float factor) {
#pragma unroll
    for (int nf = 0; nf < D / 16; ++nf) {
      wmma::store_matrix_sync(sT, acc[nf], kLdT, wmma::mem_row_major);
      __syncwarp();
      const int r = lane >> 1, c8 = (lane & 1) * 8;        // 16 rows x two halves of 8 columns
      const float* src = sT + r * kLdT + c8;
      T vals[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) vals[i] = from_float<T>(src[i] * factor);
      *reinterpret_cast<uint4*>(out_base + static_cast<int64_t>(warp * 16 + r) * row_stride + nf * 16 + c8) =
          *reinterpret_cast<const uint4*>(vals);
      __syncwarp();
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

template <typename T, int D>
cudaError_t launch_both(const AttnBwdParams& p, cudaStream_t stream) {
  const AttnParams& f = p.fwd;
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return cudaErrorNoDevice;
  auto k0 = attn_bwd_mma_kernel<T, D, 0>;
  auto k1 = attn_bwd_mma_kernel<T, D, 1>;
  constexpr size_t smem = BwdSmem<D>::total;
  static std::once_flag once[kMaxDevices];
  static cudaError_t attr[kMaxDevices];
  std::call_once(once[info->ordinal], [&] {
    cudaError_t e = cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    attr[info->ordinal] = e;
  });
  if (attr[info->ordinal] != cudaSuccess) return attr[info->ordinal];
  const long long ctas_q = static_cast<long long>(f.Sq / kR) * f.B * f.H;
  const long long ctas_k = static_cast<long long>(f.Sk / kR) * f.B * f.H;
  if (ctas_q <= 0 || ctas_k <= 0 || ctas_q > 0x7fffffffLL || ctas_k > 0x7fffffffLL) return cudaErrorInvalidValue;
  k0<<<static_cast<unsigned>(ctas_q), kThreadsMma, smem, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  k1<<<static_cast<unsigned>(ctas_k), kThreadsMma, smem, stream>>>(p);          // reads D from the first
  return cudaGetLastError();
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
