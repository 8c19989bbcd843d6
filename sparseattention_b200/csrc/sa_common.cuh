// Shared declarations of the sm_100a kernels behind the C ABI in include/sa_b200.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sa_b200.h"

namespace sa {

constexpr int kCell = 32;            // side of the cells the classifier reduces the mask to
constexpr int kStripBytes = 512;     // mask bytes one warp reads per row (32 lanes x 16 B)
constexpr int kMaxDevices = 64;      // device ordinals the per-device caches cover

// Facts about the current device, looked up once per device ordinal (thread-safe); nullptr on failure.
struct DeviceInfo {
  int ordinal;
  int sm_count;
};
const DeviceInfo* current_device_info();

// ---------------------------------------------------------------- stage 1
struct ClassifyParams {
  const uint8_t* mask;
  int64_t stride_b, stride_h, stride_q;   // elements (= bytes); stride_k == 1
  int Bu, Hu, Sq, Sk;
  int BQ, BK;
  // scratch, zero before and after a launch: per (plane, query block, strip column) a 64-bit word
  // (16 any bits, 16 not-all bits, one arrival bit per cell row) and a completed-word count per (plane,
  // query block)
  unsigned long long* words;
  unsigned int* row_counters;
  uint32_t* bits;        // optional [Bu*Hu, Sk/32, Sq]
  int32_t* full_ids;     // [Bu*Hu, nq, nk]
  int32_t* full_lens;    // [Bu*Hu, nq]
  int32_t* part_ids;
  int32_t* part_lens;
};

// Bytes of scratch for planes x nq query blocks x chunks strip columns, and where its parts start.
size_t classify_workspace_layout(int planes, int nq, int chunks, size_t* off_rows, size_t* off_words);
// Points p's scratch members into `workspace` (cleared on the stream first when asked) and launches.
cudaError_t launch_classify(ClassifyParams p, void* workspace, bool clear_first, cudaStream_t stream);
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
  int splits;                                    // >= 1; > 1 (tcgen05 kernel only): each unit's walk over its lists is cut into
                                                 // this many ranges, range s writing o / lse at batch index s * B + b
  int debug;
};

cudaError_t launch_attn_simt(const AttnParams& p, cudaStream_t stream);

// ---------------------------------------------------------------- backward of stage 2
struct AttnBwdParams {
  AttnParams fwd;                                // q, k, v, o (read), lse (read), mask, query-major lists, sizes, scale
  const void* d_o; int64_t dos[4];               // incoming gradient of O
  const float* d_lse;                            // optional incoming gradient of lse, [B,H,Sq] contiguous
  void* dq; void* dk; void* dv;
  int64_t dqs[4], dks[4], dvs[4];
  float* dsum;                                   // scratch [B,H,Sq]: per query row, sum_d dO*O (- d_lse)
  const int32_t* t_full_ids; int64_t tfis[4];    // kv-major lists: [B,H,nk,nq] / [B,H,nk] with element strides
  const int32_t* t_full_lens; int64_t tfls[3];
  const int32_t* t_part_ids; int64_t tpis[4];
  const int32_t* t_part_lens; int64_t tpls[3];
};

cudaError_t launch_transpose_lists(const int32_t* full_ids, const int32_t* full_lens, const int32_t* part_ids,
                                   const int32_t* part_lens, int planes, int nq, int nk, int32_t* t_full_ids,
                                   int32_t* t_full_lens, int32_t* t_part_ids, int32_t* t_part_lens,
                                   cudaStream_t stream);
cudaError_t launch_attn_bwd_simt(const AttnBwdParams& p, cudaStream_t stream);
// Tensor-core version (fp16 / bf16, head dim 64 or 128, unit stride along the head dim, 16-byte aligned rows).
int attn_bwd_mma_supported(const AttnBwdParams& p);
cudaError_t launch_attn_bwd_mma(const AttnBwdParams& p, cudaStream_t stream);

// Combines the partial results of a split walk (see AttnParams::splits) into o (element strides os) and lse.
cudaError_t launch_merge_splits(const void* part_o, const float* part_lse, int splits, int dtype, int B, int H, int Sq,
                                int D, void* o, const int64_t* os, float* lse, cudaStream_t stream);

// Returns 1 when the tcgen05 kernel can take this call.
int attn_tc_supported(const AttnParams& p);
// Launches the tcgen05 kernel; SA_ERR_* (negative) or 0.
int launch_attn_tc(const AttnParams& p, cudaStream_t stream);


// One CTA that waits (bounded by limit_ns) on a barrier nothing arrives on; see selftest_sm100.cu.
cudaError_t launch_bounded_wait_probe(unsigned long long limit_ns, int32_t* dev_status, unsigned long long* waited_ns,
                                      cudaStream_t stream);

}  // namespace sa
