// Backward pass of the block-sparse attention forward, on the CUDA cores (fp32 math).
//
// The reference has no backward (its README lists it as future work, README.md:61-65); this is the
// gradient of sparse_attention_kernel (sparseattention/sparse_attn_kernel.py:72-146) over the same two
// kv-block lists, from the log-sum-exp the forward emits:
//
//   P_ij  = exp(q_i.k_j * scale - lse_i)  on attended (i, j) of listed tiles, 0 elsewhere
//   D_i   = sum_d dO_id * O_id  (- the incoming gradient of lse_i, when there is one)
//   dV_j  = sum_i P_ij dO_i
//   dS_ij = P_ij * (dO_i.v_j - D_i)
//   dQ_i  = scale * sum_j dS_ij k_j          dK_j = scale * sum_i dS_ij q_i
//
// Three kernels, no atomics, so the result does not depend on the order CTAs run in:
//   transpose_lists   per (mask plane, kv block): the ascending query blocks that list it as full / as
//                     partial (a binary search in each query block's ascending lists);
//   dq kernel         one CTA per 32 query rows, a quad of threads per row, walking the row's lists exactly
//                     like the forward (full list without the mask, partial list with it); also writes D;
//   dkdv kernel       one CTA per 32 kv rows, a quad per row, walking the transposed lists.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sa_common.cuh"

namespace sa {
namespace {

constexpr int kRows = 32;       // rows per CTA (query rows in the dq kernel, kv rows in the dkdv kernel)
constexpr int kChunk = 32;      // rows of the other side staged per step
constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// ---------------------------------------------------------------------------------------------
// kv-major lists from query-major lists.  One CTA per (plane, kv block j); thread t looks query block
// i = i0 + t up: j is in i's full list, in its partial list, or in neither (both lists ascend).
__device__ __forceinline__ bool listed(const int32_t* ids, int len, int j) {
  int lo = 0, hi = len;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    const int v = ids[mid];
    if (v < j) lo = mid + 1; else hi = mid;
  }
  return lo < len && ids[lo] == j;
}

__global__ void __launch_bounds__(kThreads)
transpose_lists_kernel(const int32_t* __restrict__ full_ids, const int32_t* __restrict__ full_lens,
                       const int32_t* __restrict__ part_ids, const int32_t* __restrict__ part_lens,
                       const int nq, const int nk,
                       int32_t* __restrict__ t_full_ids, int32_t* __restrict__ t_full_lens,
                       int32_t* __restrict__ t_part_ids, int32_t* __restrict__ t_part_lens) {
  __shared__ int s_full[kThreads / 32], s_part[kThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int plane = blockIdx.x / nk, j = blockIdx.x % nk;
  int32_t* f_out = t_full_ids + static_cast<int64_t>(blockIdx.x) * nq;
  int32_t* p_out = t_part_ids + static_cast<int64_t>(blockIdx.x) * nq;
  const uint32_t lt_mask = (1u << lane) - 1u;
  int nf = 0, np = 0;
  for (int i0 = 0; i0 < nq; i0 += kThreads) {
    const int i = i0 + tid;
    bool is_full = false, is_part = false;
    if (i < nq) {
      const int64_t row = static_cast<int64_t>(plane) * nq + i;
      const int lf = min(max(full_lens[row], 0), nk), lp = min(max(part_lens[row], 0), nk);
      is_full = listed(full_ids + row * nk, lf, j);
      is_part = !is_full && listed(part_ids + row * nk, lp, j);
    }
    const uint32_t bf = __ballot_sync(0xffffffffu, is_full);
    const uint32_t bp = __ballot_sync(0xffffffffu, is_part);
    if (lane == 0) { s_full[warp] = __popc(bf); s_part[warp] = __popc(bp); }
    __syncthreads();
    int off_f = nf, off_p = np, tot_f = 0, tot_p = 0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) {
      if (w < warp) { off_f += s_full[w]; off_p += s_part[w]; }
      tot_f += s_full[w];
      tot_p += s_part[w];
    }
    if (is_full) f_out[off_f + __popc(bf & lt_mask)] = i;
    if (is_part) p_out[off_p + __popc(bp & lt_mask)] = i;
    nf += tot_f;
    np += tot_p;
    __syncthreads();
  }
  for (int t = nf + tid; t < nq; t += kThreads) f_out[t] = -1;
  for (int t = np + tid; t < nq; t += kThreads) p_out[t] = -1;
  if (tid == 0) {
    t_full_lens[blockIdx.x] = nf;
    t_part_lens[blockIdx.x] = np;
  }
}

// ---------------------------------------------------------------------------------------------
// dQ (and D): the forward's walk over the lists of a query row.
template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
attn_bwd_dq_kernel(const AttnBwdParams p) {
  constexpr int DQ = D / 4;
  __shared__ float Ks[kChunk][D];
  __shared__ float Vs[kChunk][D];
  const AttnParams& f = p.fwd;

  const int tid = threadIdx.x;
  const int r = tid >> 2, ql = tid & 3;
  const int row_groups = f.Sq / kRows;
  const int row = static_cast<int>(blockIdx.x % row_groups) * kRows + r;
  const int bh = static_cast<int>(blockIdx.x / row_groups);
  const int b = bh / f.H, h = bh % f.H;
  const int qblk = row / f.BQ;
  const int nk = f.Sk / f.BK;

  const T* q = static_cast<const T*>(f.q) + b * f.qs[0] + h * f.qs[1] + static_cast<int64_t>(row) * f.qs[2];
  const T* o = static_cast<const T*>(f.o) + b * f.os[0] + h * f.os[1] + static_cast<int64_t>(row) * f.os[2];
  const T* g = static_cast<const T*>(p.d_o) + b * p.dos[0] + h * p.dos[1] + static_cast<int64_t>(row) * p.dos[2];
  const T* kbase = static_cast<const T*>(f.k) + b * f.ks[0] + h * f.ks[1];
  const T* vbase = static_cast<const T*>(f.v) + b * f.vs[0] + h * f.vs[1];
  const uint8_t* mrow = f.mask + b * f.ms[0] + h * f.ms[1] + static_cast<int64_t>(row) * f.ms[2];
  const int64_t stat = (static_cast<int64_t>(b) * f.H + h) * f.Sq + row;

  float qv[DQ], gv[DQ], acc[DQ];
  float dsum = 0.f;
#pragma unroll
  for (int j = 0; j < DQ; ++j) {
    qv[j] = to_f32<T>(q[static_cast<int64_t>(4 * j + ql) * f.qs[3]]);
    gv[j] = to_f32<T>(g[static_cast<int64_t>(4 * j + ql) * p.dos[3]]);
    dsum = fmaf(gv[j], to_f32<T>(o[static_cast<int64_t>(4 * j + ql) * f.os[3]]), dsum);
    acc[j] = 0.f;
  }
  dsum = quad_sum(dsum);
  if (p.d_lse != nullptr) dsum -= p.d_lse[stat];
  if (ql == 0) p.dsum[stat] = dsum;
  const float lse = f.lse[stat];
  const bool live = lse > -INFINITY;               // a row with no attended key has no gradient
  const float lse2 = lse * kLog2e;

#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const bool masked = pass == 1;
    const int32_t* ids = masked
        ? f.part_ids + b * f.pis[0] + h * f.pis[1] + static_cast<int64_t>(qblk) * f.pis[2]
        : f.full_ids + b * f.fis[0] + h * f.fis[1] + static_cast<int64_t>(qblk) * f.fis[2];
    const int64_t id_stride = masked ? f.pis[3] : f.fis[3];
    const int n_given = masked
        ? f.part_lens[b * f.pls[0] + h * f.pls[1] + static_cast<int64_t>(qblk) * f.pls[2]]
        : f.full_lens[b * f.fls[0] + h * f.fls[1] + static_cast<int64_t>(qblk) * f.fls[2]];
    const int n = min(max(n_given, 0), nk);
#pragma unroll 1
    for (int t = 0; t < n; ++t) {
      const int id = ids[t * id_stride];
      if (id < 0 || id >= nk) {
        if (tid == 0 && f.dev_status != nullptr) atomicMax(f.dev_status, SA_DEV_BAD_INDEX);
        continue;
      }
#pragma unroll 1
      for (int sub = 0; sub < f.BK; sub += kChunk) {
        const int kv0 = id * f.BK + sub;
        __syncthreads();
        for (int e = tid; e < kChunk * D; e += kThreads) {
          const int c = e / D, d = e % D;
          Ks[c][d] = to_f32<T>(kbase[static_cast<int64_t>(kv0 + c) * f.ks[2] + d * f.ks[3]]);
          Vs[c][d] = to_f32<T>(vbase[static_cast<int64_t>(kv0 + c) * f.vs[2] + d * f.vs[3]]);
        }
        __syncthreads();
#pragma unroll 4
        for (int c = 0; c < kChunk; ++c) {
          float s = 0.f, dp = 0.f;
#pragma unroll
          for (int j = 0; j < DQ; ++j) {
            s = fmaf(qv[j], Ks[c][4 * j + ql], s);
            dp = fmaf(gv[j], Vs[c][4 * j + ql], dp);
          }
          s = quad_sum(s);
          dp = quad_sum(dp);
          const bool attend = live && !(masked && mrow[static_cast<int64_t>(kv0 + c) * f.ms[3]] == 0);
          const float pe = attend ? exp2f(s * f.scale_log2 - lse2) : 0.f;
          const float ds = pe * (dp - dsum);
#pragma unroll
          for (int j = 0; j < DQ; ++j) acc[j] = fmaf(ds, Ks[c][4 * j + ql], acc[j]);
        }
      }
    }
  }
  const float scale = f.scale_log2 * kLn2;
  T* dq = static_cast<T*>(p.dq) + b * p.dqs[0] + h * p.dqs[1] + static_cast<int64_t>(row) * p.dqs[2];
#pragma unroll
  for (int j = 0; j < DQ; ++j) dq[static_cast<int64_t>(4 * j + ql) * p.dqs[3]] = from_f32<T>(acc[j] * scale);
}

// ---------------------------------------------------------------------------------------------
// dK, dV: a kv row walks the query blocks that list its kv block (transposed lists).
template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
attn_bwd_dkdv_kernel(const AttnBwdParams p) {
  constexpr int DQ = D / 4;
  __shared__ float Qs[kChunk][D];
  __shared__ float Gs[kChunk][D];
  __shared__ float s_lse2[kChunk], s_dsum[kChunk];
  const AttnParams& f = p.fwd;

  const int tid = threadIdx.x;
  const int r = tid >> 2, ql = tid & 3;
  const int row_groups = f.Sk / kRows;
  const int kvrow = static_cast<int>(blockIdx.x % row_groups) * kRows + r;
  const int bh = static_cast<int>(blockIdx.x / row_groups);
  const int b = bh / f.H, h = bh % f.H;
  const int kvblk = kvrow / f.BK;
  const int nq = f.Sq / f.BQ;

  const T* kr = static_cast<const T*>(f.k) + b * f.ks[0] + h * f.ks[1] + static_cast<int64_t>(kvrow) * f.ks[2];
  const T* vr = static_cast<const T*>(f.v) + b * f.vs[0] + h * f.vs[1] + static_cast<int64_t>(kvrow) * f.vs[2];
  const T* qbase = static_cast<const T*>(f.q) + b * f.qs[0] + h * f.qs[1];
  const T* gbase = static_cast<const T*>(p.d_o) + b * p.dos[0] + h * p.dos[1];
  const uint8_t* mcol = f.mask + b * f.ms[0] + h * f.ms[1] + static_cast<int64_t>(kvrow) * f.ms[3];
  const int64_t stat0 = (static_cast<int64_t>(b) * f.H + h) * f.Sq;

  float kv[DQ], vv[DQ], dk[DQ], dv[DQ];
#pragma unroll
  for (int j = 0; j < DQ; ++j) {
    kv[j] = to_f32<T>(kr[static_cast<int64_t>(4 * j + ql) * f.ks[3]]);
    vv[j] = to_f32<T>(vr[static_cast<int64_t>(4 * j + ql) * f.vs[3]]);
    dk[j] = dv[j] = 0.f;
  }

#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const bool masked = pass == 1;
    const int32_t* ids = masked
        ? p.t_part_ids + b * p.tpis[0] + h * p.tpis[1] + static_cast<int64_t>(kvblk) * p.tpis[2]
        : p.t_full_ids + b * p.tfis[0] + h * p.tfis[1] + static_cast<int64_t>(kvblk) * p.tfis[2];
    const int64_t id_stride = masked ? p.tpis[3] : p.tfis[3];
    const int n_given = masked
        ? p.t_part_lens[b * p.tpls[0] + h * p.tpls[1] + static_cast<int64_t>(kvblk) * p.tpls[2]]
        : p.t_full_lens[b * p.tfls[0] + h * p.tfls[1] + static_cast<int64_t>(kvblk) * p.tfls[2]];
    const int n = min(max(n_given, 0), nq);
#pragma unroll 1
    for (int t = 0; t < n; ++t) {
      const int id = ids[t * id_stride];
      if (id < 0 || id >= nq) {
        if (tid == 0 && f.dev_status != nullptr) atomicMax(f.dev_status, SA_DEV_BAD_INDEX);
        continue;
      }
#pragma unroll 1
      for (int sub = 0; sub < f.BQ; sub += kChunk) {
        const int q0 = id * f.BQ + sub;
        __syncthreads();
        for (int e = tid; e < kChunk * D; e += kThreads) {
          const int c = e / D, d = e % D;
          Qs[c][d] = to_f32<T>(qbase[static_cast<int64_t>(q0 + c) * f.qs[2] + d * f.qs[3]]);
          Gs[c][d] = to_f32<T>(gbase[static_cast<int64_t>(q0 + c) * p.dos[2] + d * p.dos[3]]);
        }
        if (tid < kChunk) {
          s_lse2[tid] = f.lse[stat0 + q0 + tid] * kLog2e;
          s_dsum[tid] = p.dsum[stat0 + q0 + tid];
        }
        __syncthreads();
#pragma unroll 4
        for (int c = 0; c < kChunk; ++c) {
          float s = 0.f, dp = 0.f;
#pragma unroll
          for (int j = 0; j < DQ; ++j) {
            s = fmaf(kv[j], Qs[c][4 * j + ql], s);
            dp = fmaf(vv[j], Gs[c][4 * j + ql], dp);
          }
          s = quad_sum(s);
          dp = quad_sum(dp);
          const bool attend = s_lse2[c] > -INFINITY &&
                              !(masked && mcol[static_cast<int64_t>(q0 + c) * f.ms[2]] == 0);
          const float pe = attend ? exp2f(s * f.scale_log2 - s_lse2[c]) : 0.f;
          const float ds = pe * (dp - s_dsum[c]);
#pragma unroll
          for (int j = 0; j < DQ; ++j) {
            dv[j] = fmaf(pe, Gs[c][4 * j + ql], dv[j]);
            dk[j] = fmaf(ds, Qs[c][4 * j + ql], dk[j]);
          }
        }
      }
    }
  }
  const float scale = f.scale_log2 * kLn2;
  T* dko = static_cast<T*>(p.dk) + b * p.dks[0] + h * p.dks[1] + static_cast<int64_t>(kvrow) * p.dks[2];
  T* dvo = static_cast<T*>(p.dv) + b * p.dvs[0] + h * p.dvs[1] + static_cast<int64_t>(kvrow) * p.dvs[2];
#pragma unroll
  for (int j = 0; j < DQ; ++j) {
    dko[static_cast<int64_t>(4 * j + ql) * p.dks[3]] = from_f32<T>(dk[j] * scale);
    dvo[static_cast<int64_t>(4 * j + ql) * p.dvs[3]] = from_f32<T>(dv[j]);
  }
}

template <typename T, int D>
cudaError_t launch_both(const AttnBwdParams& p, cudaStream_t stream) {
  const AttnParams& f = p.fwd;
  const long long ctas_q = static_cast<long long>(f.Sq / kRows) * f.B * f.H;
  const long long ctas_k = static_cast<long long>(f.Sk / kRows) * f.B * f.H;
  if (ctas_q <= 0 || ctas_k <= 0 || ctas_q > 0x7fffffffLL || ctas_k > 0x7fffffffLL) return cudaErrorInvalidValue;
  attn_bwd_dq_kernel<T, D><<<static_cast<unsigned>(ctas_q), kThreads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  attn_bwd_dkdv_kernel<T, D><<<static_cast<unsigned>(ctas_k), kThreads, 0, stream>>>(p);   // reads D from the first
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_for_dtype(const AttnBwdParams& p, cudaStream_t stream) {
  switch (p.fwd.D) {
    case 16:  return launch_both<T, 16>(p, stream);
    case 32:  return launch_both<T, 32>(p, stream);
    case 64:  return launch_both<T, 64>(p, stream);
    case 128: return launch_both<T, 128>(p, stream);
    default:  return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_transpose_lists(const int32_t* full_ids, const int32_t* full_lens, const int32_t* part_ids,
                                   const int32_t* part_lens, int planes, int nq, int nk, int32_t* t_full_ids,
                                   int32_t* t_full_lens, int32_t* t_part_ids, int32_t* t_part_lens,
                                   cudaStream_t stream) {
  transpose_lists_kernel<<<static_cast<unsigned>(planes * nk), kThreads, 0, stream>>>(
      full_ids, full_lens, part_ids, part_lens, nq, nk, t_full_ids, t_full_lens, t_part_ids, t_part_lens);
  return cudaGetLastError();
}

cudaError_t launch_attn_bwd_simt(const AttnBwdParams& p, cudaStream_t stream) {
  switch (p.fwd.dtype) {
    case SA_DTYPE_F32:  return launch_for_dtype<float>(p, stream);
    case SA_DTYPE_F16:  return launch_for_dtype<__half>(p, stream);
    case SA_DTYPE_BF16: return launch_for_dtype<__nv_bfloat16>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace sa
