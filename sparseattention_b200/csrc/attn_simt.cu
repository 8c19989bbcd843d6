// Stage 2, generic kernel: block-sparse attention forward on the CUDA cores.
//
// Same algorithm as sparseattention/sparse_attn_kernel.py:72-146 (+ inner loop 10-63):
// per query block, loop A over the full list without the mask, loop B over the partial
// list with the boolean mask applied as -inf, online softmax in base 2 with fp32 running
// max / sum / accumulator, P rounded to the V dtype before P.V (line 61), O = acc / l.
// It takes any dtype (fp32 / fp16 / bf16), any strides (0 included), head dims 16, 32, 64
// and 128 and block sizes that are multiples of 32, reads the byte mask
// directly, and is the path for shapes the tcgen05 kernel does not cover.  Rows without
// any attended key come out as 0.
//
// Work split: one CTA of 128 threads per 32 query rows of one (batch, head); a quad of
// threads owns a row, each thread holding the d = 4j + quad_lane elements of q and acc.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sa_common.cuh"

namespace sa {
namespace {

constexpr int kRows = 32;       // query rows per CTA
constexpr int kChunk = 32;      // kv rows staged per step
constexpr int kThreads = 128;

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
attn_simt_kernel(const AttnParams p) {
  constexpr int DQ = D / 4;
  __shared__ float Ks[kChunk][D];
  __shared__ float Vs[kChunk][D];

  const int tid = threadIdx.x;
  const int r = tid >> 2, ql = tid & 3;
  const int row_groups = p.Sq / kRows;                   // 1-D grid: (batch * head, group of 32 query rows)
  const int row = static_cast<int>(blockIdx.x % row_groups) * kRows + r;
  const int bh = static_cast<int>(blockIdx.x / row_groups);
  const int b = bh / p.H, h = bh % p.H;
  const int qblk = row / p.BQ;
  const int nk = p.Sk / p.BK;

  const T* q = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + static_cast<int64_t>(row) * p.qs[2];
  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
  const uint8_t* mrow = p.mask + b * p.ms[0] + h * p.ms[1] + static_cast<int64_t>(row) * p.ms[2];

  float qv[DQ], acc[DQ];
#pragma unroll
  for (int j = 0; j < DQ; ++j) {
    qv[j] = to_f32<T>(q[static_cast<int64_t>(4 * j + ql) * p.qs[3]]);   // sparse_attn_kernel.py:98-101
    acc[j] = 0.f;                                                        // line 105
  }
  float m = -INFINITY, l = 0.f;                                          // lines 103-104

#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const bool masked = pass == 1;
    const int32_t* ids = masked
        ? p.part_ids + b * p.pis[0] + h * p.pis[1] + static_cast<int64_t>(qblk) * p.pis[2]
        : p.full_ids + b * p.fis[0] + h * p.fis[1] + static_cast<int64_t>(qblk) * p.fis[2];
    const int64_t id_stride = masked ? p.pis[3] : p.fis[3];
    const int n_given = masked
        ? p.part_lens[b * p.pls[0] + h * p.pls[1] + static_cast<int64_t>(qblk) * p.pls[2]]   // line 127
        : p.full_lens[b * p.fls[0] + h * p.fls[1] + static_cast<int64_t>(qblk) * p.fls[2]];  // line 107
    // A caller-supplied length outside [0, nk] would walk the id list out of bounds: it is clamped
    // (as the tensor-core kernel does) and reported.
    const int n = min(max(n_given, 0), nk);
    if (n != n_given && tid == 0 && p.dev_status != nullptr) atomicMax(p.dev_status, SA_DEV_BAD_INDEX);
#pragma unroll 1
    for (int t = 0; t < n; ++t) {
      const int id = ids[t * id_stride];                                 // line 33
      if (id < 0 || id >= nk) {                                          // uniform across the CTA
        if (tid == 0 && p.dev_status != nullptr) atomicMax(p.dev_status, SA_DEV_BAD_INDEX);
        continue;
      }
#pragma unroll 1
      for (int sub = 0; sub < p.BK; sub += kChunk) {
        const int kv0 = id * p.BK + sub;
        __syncthreads();
        for (int e = tid; e < kChunk * D; e += kThreads) {
          const int c = e / D, d = e % D;
          Ks[c][d] = to_f32<T>(kbase[static_cast<int64_t>(kv0 + c) * p.ks[2] + d * p.ks[3]]);
          Vs[c][d] = to_f32<T>(vbase[static_cast<int64_t>(kv0 + c) * p.vs[2] + d * p.vs[3]]);
        }
        __syncthreads();

        float s[kChunk];
        float tile_max = -INFINITY;
#pragma unroll
        for (int c = 0; c < kChunk; ++c) {
          float part = 0.f;
#pragma unroll
          for (int j = 0; j < DQ; ++j) part = fmaf(qv[j], Ks[c][4 * j + ql], part);   // line 40
          part += __shfl_xor_sync(0xffffffffu, part, 1);
          part += __shfl_xor_sync(0xffffffffu, part, 2);
          float sc = part * p.scale_log2;                                               // lines 47 / 51
          if (masked && mrow[static_cast<int64_t>(kv0 + c) * p.ms[3]] == 0) sc = -INFINITY;  // line 47
          s[c] = sc;
          tile_max = fmaxf(tile_max, sc);
        }
        const float m_new = fmaxf(m, tile_max);                                         // lines 48 / 50
        const float ref = (m_new == -INFINITY) ? 0.f : m_new;      // guard the reference lacks (line 53)
        const float alpha = (m == -INFINITY) ? 1.f : exp2f(m - ref);                    // line 55
        float row_sum = 0.f;
#pragma unroll
        for (int c = 0; c < kChunk; ++c) {
          const float pe = exp2f(s[c] - ref);                                           // line 54
          row_sum += pe;
          s[c] = to_f32<T>(from_f32<T>(pe));                                            // line 61 cast
        }
        l = l * alpha + row_sum;                                                        // line 57
        m = m_new;                                                                      // line 56
#pragma unroll
        for (int j = 0; j < DQ; ++j) acc[j] *= alpha;                                   // line 58
#pragma unroll
        for (int c = 0; c < kChunk; ++c) {
#pragma unroll
          for (int j = 0; j < DQ; ++j) acc[j] = fmaf(s[c], Vs[c][4 * j + ql], acc[j]);  // line 61
        }
      }
    }
  }

  const float inv = l > 0.f ? 1.f / l : 0.f;                                            // line 144
  if (p.lse != nullptr && ql == 0)                 // m and l are in base 2 (scale folded, line 152)
    p.lse[(static_cast<int64_t>(b) * p.H + h) * p.Sq + row] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
  T* o = static_cast<T*>(p.o) + b * p.os[0] + h * p.os[1] + static_cast<int64_t>(row) * p.os[2];
#pragma unroll
  for (int j = 0; j < DQ; ++j) o[static_cast<int64_t>(4 * j + ql) * p.os[3]] = from_f32<T>(acc[j] * inv);  // line 146
}

template <typename T>
cudaError_t launch_for_dtype(const AttnParams& p, cudaStream_t stream) {
  const long long ctas = static_cast<long long>(p.Sq / kRows) * p.B * p.H;
  if (ctas <= 0 || ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  dim3 grid(static_cast<unsigned>(ctas));
  switch (p.D) {
    case 16:  attn_simt_kernel<T, 16><<<grid, kThreads, 0, stream>>>(p); break;
    case 32:  attn_simt_kernel<T, 32><<<grid, kThreads, 0, stream>>>(p); break;
    case 64:  attn_simt_kernel<T, 64><<<grid, kThreads, 0, stream>>>(p); break;
    case 128: attn_simt_kernel<T, 128><<<grid, kThreads, 0, stream>>>(p); break;
    default:  return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_attn_simt(const AttnParams& p, cudaStream_t stream) {
  switch (p.dtype) {
    case SA_DTYPE_F32:  return launch_for_dtype<float>(p, stream);
    case SA_DTYPE_F16:  return launch_for_dtype<__half>(p, stream);
    case SA_DTYPE_BF16: return launch_for_dtype<__nv_bfloat16>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace sa
