// Shared declarations of the sm_100a kernels behind the C ABI in include/sa_b200.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sa_b200.h"

namespace sa {

constexpr int kCell = 32;            // side of the cells the classifier reduces the mask to
constexpr int kStripBytes = 512;     // mask bytes one warp reads per row (32 lanes x 16 B)

// ---------------------------------------------------------------- stage 1
struct ClassifyParams {
  const uint8_t* mask;
  int64_t stride_b, stride_h, stride_q;   // elements (= bytes); stride_k == 1
  int Bu, Hu, Sq, Sk;
  int BQ, BK;
  uint8_t* cells;        // [Bu*Hu, Sq/32, Sk/32] flag bytes: bit0 = any True, bit1 = all True
  uint32_t* bits;        // optional [Bu*Hu, Sk/32, Sq]
  int32_t* full_ids;     // [Bu*Hu, nq, nk]
  int32_t* full_lens;    // [Bu*Hu, nq]
  int32_t* part_ids;
  int32_t* part_lens;
};

cudaError_t launch_classify(const ClassifyParams& p, cudaStream_t stream);
// Lists of query blocks `ratio` times shorter -> lists of the tall blocks (p_out: output pointers only).
cudaError_t launch_merge_lists(const int32_t* full_ids_in, const int32_t* full_lens_in, const int32_t* part_ids_in,
                               const int32_t* part_lens_in, int planes, int nq_out, int nk, int ratio,
                               int bq_in, int bk, ClassifyParams p_out, cudaStream_t stream);

// ---------------------------------------------------------------- stage 2
struct AttnParams {
  const void* q; const void* k; const void* v; void* o;
  int64_t qs[4], ks[4], vs[4], os[4];            // element strides (b,h,s,d)
  const uint8_t* mask; int64_t ms[4];
  const uint32_t* bits; int64_t bits_sb, bits_sh;  // word strides over (b,h)
  const int32_t* full_ids; int64_t fis[4];
  const int32_t* full_lens; int64_t fls[3];
  const int32_t* part_ids; int64_t pis[4];
  const int32_t* part_lens; int64_t pls[3];
  int B, H, Sq, Sk, D, BQ, BK;
  int dtype;
  float scale_log2;
  float* lse;                                    // optional [B,H,Sq] contiguous: natural-log sum of exp of the scaled scores
  int32_t* dev_status;
  int32_t* tile_counter;                         // zeroed device word for the tile scheduler, or null (static order)
  int debug;
};

cudaError_t launch_attn_simt(const AttnParams& p, cudaStream_t stream);

// Returns 1 when the tcgen05 kernel can take this call.
int attn_tc_supported(const AttnParams& p);
// Launches the tcgen05 kernel; SA_ERR_* (negative) or 0.
int launch_attn_tc(const AttnParams& p, cudaStream_t stream);

}  // namespace sa
