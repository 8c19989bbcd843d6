// Stage 1: block classifier for a dense boolean attention mask (HBM-bound).
//
// Replaces sparseattention/mask_utils.py:47-107 (_compute_mask_inner + its launcher).
// The reference walks the kv blocks of one query block serially in one program and
// re-reads an expanded mask once per head; here every distinct mask byte is read
// exactly once with 16-byte loads:
//
//   cells kernel   one warp per 32-row x 512-column strip: each lane streams 32 rows of
//                  16 bytes, reduces them to "any / all" flags of the 32x32 cells (a lane
//                  pair per cell) and, optionally, emits the packed bit-plane stage 2 reads.
//   lists kernel   one CTA per (mask plane, query block), launched as a programmatic
//                  dependent of the cells kernel: folds the cell flags of each
//                  BLOCK_Q x BLOCK_K tile, ballots the full / partial predicates and writes the
//                  ascending id lists by a popcount prefix (order of mask_utils.py:66-79),
//                  tails filled with -1.
#include "sa_common.cuh"

namespace sa {
namespace {

__device__ __forceinline__ uint4 ld_stream_16(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// 4 mask bytes -> 4 bits (bit i = byte i non-zero).
__device__ __forceinline__ uint32_t nibble_of(uint32_t w) {
  uint32_t nz = (((w & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w) >> 7;
  nz &= 0x01010101u;
  return (nz * 0x01020408u) >> 24;   // gathers bits 0,8,16,24 into bits 0..3
}

__device__ __forceinline__ uint32_t half_word_of(const uint4& v) {
  return nibble_of(v.x) | (nibble_of(v.y) << 4) | (nibble_of(v.z) << 8) | (nibble_of(v.w) << 12);
}

constexpr int kCellsThreads = 256;

__global__ void __launch_bounds__(kCellsThreads)
classify_cells_kernel(const ClassifyParams p, const int chunks_per_row, const long long n_strips) {
  // lets the lists kernel be scheduled early; it waits for this grid to complete before reading
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * kCellsThreads + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * kCellsThreads) >> 5;
  const int row_cells = p.Sq / kCell;
  const int col_cells = p.Sk / kCell;
  const int odd = lane & 1;

  for (long long strip = warp0; strip < n_strips; strip += n_warps) {
    const int chunk = static_cast<int>(strip % chunks_per_row);
    const long long t = strip / chunks_per_row;
    const int rc = static_cast<int>(t % row_cells);
    const int plane = static_cast<int>(t / row_cells);
    const int b = plane / p.Hu, h = plane % p.Hu;
    const int col = chunk * kStripBytes + lane * 16;
    const bool active = col < p.Sk;
    const uint8_t* base = p.mask + b * p.stride_b + h * p.stride_h +
                          static_cast<int64_t>(rc) * kCell * p.stride_q + col;

    uint32_t and_acc = 0xffffu, or_acc = 0u;
    uint32_t keep[16];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint4 v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        v[r] = active ? ld_stream_16(base + static_cast<int64_t>(g * 8 + r) * p.stride_q)
                      : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int row = g * 8 + r;
        const uint32_t hb = half_word_of(v[r]);
        and_acc &= hb;
        or_acc |= hb;
        const uint32_t other = __shfl_xor_sync(0xffffffffu, hb, 1);
        const uint32_t word = odd ? (other | (hb << 16)) : (hb | (other << 16));
        // even lanes keep rows 0..15 of the cell, odd lanes rows 16..31
        if ((row >> 4) == 0) { if (!odd) keep[row & 15] = word; }
        else                 { if (odd)  keep[row & 15] = word; }
      }
    }
    const uint32_t and_all = and_acc & __shfl_xor_sync(0xffffffffu, and_acc, 1);
    const uint32_t or_any = or_acc | __shfl_xor_sync(0xffffffffu, or_acc, 1);
    if (active) {
      const int kb = chunk * (kStripBytes / kCell) + (lane >> 1);
      if (!odd) {
        const uint8_t flag = static_cast<uint8_t>((or_any != 0u ? 1u : 0u) | (and_all == 0xffffu ? 2u : 0u));
        p.cells[(static_cast<int64_t>(plane) * row_cells + rc) * col_cells + kb] = flag;
      }
      if (p.bits != nullptr) {
        uint4* dst = reinterpret_cast<uint4*>(
            p.bits + (static_cast<int64_t>(plane) * col_cells + kb) * p.Sq + rc * kCell + odd * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          dst[i] = make_uint4(keep[4 * i], keep[4 * i + 1], keep[4 * i + 2], keep[4 * i + 3]);
      }
    }
  }
}

constexpr int kListsThreads = 128;

// Folds the flags of the BLOCK_Q x BLOCK_K tiles of one query block (flags[y * flag_pitch + x] for the
// 32 x 32 cell (y, x) of the block: bit 0 = any True, bit 1 = all True) and writes the block's two
// ascending id lists, their -1 tails and lengths.  128 tiles per pass, one per thread; the order of
// the ids (ascending kv block, mask_utils.py:66-79) comes from a ballot within each warp and a prefix
// over the four warps.  Called by all kListsThreads threads of a CTA.
__device__ __forceinline__ void build_lists(const ClassifyParams& p, const uint8_t* flags, int64_t flag_pitch,
                                            int row, int* s_full, int* s_part) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nk = p.Sk / p.BK;
  const int rq = p.BQ / kCell, rk = p.BK / kCell;
  int32_t* f_out = p.full_ids + static_cast<int64_t>(row) * nk;
  int32_t* p_out = p.part_ids + static_cast<int64_t>(row) * nk;
  const uint32_t lt_mask = (1u << lane) - 1u;
  int nf = 0, np = 0;
  for (int j0 = 0; j0 < nk; j0 += kListsThreads) {
    const int j = j0 + tid;
    uint32_t any = 0u, all = 2u;
    if (j < nk) {
      for (int y = 0; y < rq; ++y) {
        const uint8_t* c = flags + static_cast<int64_t>(y) * flag_pitch + static_cast<int64_t>(j) * rk;
        for (int x = 0; x < rk; ++x) {
          const uint32_t f = c[x];
          any |= f;
          all &= f;
        }
      }
    }
    const bool is_full = (j < nk) && (all & 2u);                 // count == BQ*BK  (mask_utils.py:72)
    const bool is_part = (j < nk) && !is_full && (any & 1u);     // 0 < count       (mask_utils.py:76)
    const uint32_t bf = __ballot_sync(0xffffffffu, is_full);
    const uint32_t bp = __ballot_sync(0xffffffffu, is_part);
    if (lane == 0) { s_full[warp] = __popc(bf); s_part[warp] = __popc(bp); }
    __syncthreads();
    int off_f = nf, off_p = np, tot_f = 0, tot_p = 0;
#pragma unroll
    for (int w = 0; w < kListsThreads / 32; ++w) {
      if (w < warp) { off_f += s_full[w]; off_p += s_part[w]; }
      tot_f += s_full[w];
      tot_p += s_part[w];
    }
    if (is_full) f_out[off_f + __popc(bf & lt_mask)] = j;
    if (is_part) p_out[off_p + __popc(bp & lt_mask)] = j;
    nf += tot_f;
    np += tot_p;
    __syncthreads();
  }
  for (int t = nf + tid; t < nk; t += kListsThreads) f_out[t] = -1;
  for (int t = np + tid; t < nk; t += kListsThreads) p_out[t] = -1;
  if (tid == 0) {
    p.full_lens[row] = nf;                                       // mask_utils.py:81
    p.part_lens[row] = np;                                       // mask_utils.py:82
  }
}

// One CTA per (mask plane, query block).
__global__ void __launch_bounds__(kListsThreads)
compact_lists_kernel(const ClassifyParams p, const int n_rows) {
  asm volatile("griddepcontrol.wait;" ::: "memory");     // the cell flags of the streaming kernel are complete
  __shared__ int s_full[kListsThreads / 32], s_part[kListsThreads / 32];
  const int row = blockIdx.x;                                       // (plane, query block)
  if (row >= n_rows) return;
  const int nq = p.Sq / p.BQ, rq = p.BQ / kCell;
  const int row_cells = p.Sq / kCell, col_cells = p.Sk / kCell;
  const int plane = row / nq, i = row % nq;
  const uint8_t* cells = p.cells + (static_cast<int64_t>(plane) * row_cells + static_cast<int64_t>(i) * rq) * col_cells;
  build_lists(p, cells, col_cells, row, s_full, s_part);
}

// Lists of short query blocks -> lists of the tall query blocks that contain `ratio` of them each.
// One CTA per tall block: the short blocks' lists are scattered into per-(short block, kv block)
// flags in shared memory (3 = in the full list, 1 = in the partial list, 0 = not listed), which
// build_lists folds like cell flags: full for the tall block if full for every short block,
// partial if listed by any.  Dynamic shared memory: ratio * nk bytes.
//
// With a bit plane (p_out.bits, [planes, Sk/32, Sq], made from the mask) the kernel also makes the
// plane say what the short lists say, for the tiles stage 2 will read it for (the tall partial ones):
// rows of a short block that does not list the kv block become all False, rows of one that lists it
// as full become all True.  For lists that were derived from the same mask this rewrites words with
// the value they already have; for lists a caller has pruned or widened it is what keeps the result
// equal to walking the short lists (sparse_attn_kernel.py:113-142).  bq_in, bk: the short lists' block sizes.
__global__ void __launch_bounds__(kListsThreads)
merge_lists_kernel(const ClassifyParams p_out, const int32_t* __restrict__ full_ids_in,
                   const int32_t* __restrict__ full_lens_in, const int32_t* __restrict__ part_ids_in,
                   const int32_t* __restrict__ part_lens_in, const int nq_out, const int nk, const int ratio,
                   const int bq_in, const int bk) {
  extern __shared__ uint8_t s_listed[];
  __shared__ int s_full[kListsThreads / 32], s_part[kListsThreads / 32];
  const int tid = threadIdx.x;
  const int row = blockIdx.x;                                       // (plane, tall query block)
  const int plane = row / nq_out, i = row % nq_out;
  for (int t = tid; t < ratio * nk; t += kListsThreads) s_listed[t] = 0;
  __syncthreads();
  for (int s = 0; s < ratio; ++s) {
    const int64_t row_in = (static_cast<int64_t>(plane) * nq_out + i) * ratio + s;
    const int nf = min(max(full_lens_in[row_in], 0), nk), np = min(max(part_lens_in[row_in], 0), nk);
    for (int t = tid; t < nf; t += kListsThreads) {
      const int id = full_ids_in[row_in * nk + t];
      if (static_cast<unsigned>(id) < static_cast<unsigned>(nk)) s_listed[s * nk + id] = 3;
    }
    for (int t = tid; t < np; t += kListsThreads) {
      const int id = part_ids_in[row_in * nk + t];
      if (static_cast<unsigned>(id) < static_cast<unsigned>(nk)) s_listed[s * nk + id] = 1;
    }
  }
  __syncthreads();
  build_lists(p_out, s_listed, nk, row, s_full, s_part);
  if (p_out.bits == nullptr) return;
  const int lane = tid & 31, warp = tid >> 5;
  const int wpb = bk / kCell;                                       // 32-column word groups per kv block
  uint32_t* plane_bits = p_out.bits + static_cast<int64_t>(plane) * (static_cast<int64_t>(nk) * wpb) * p_out.Sq;
  const int row0 = i * ratio * bq_in;                               // first query row of the tall block
  for (int j = warp; j < nk; j += kListsThreads / 32) {
    uint32_t any = 0u, all = 2u;
    for (int s = 0; s < ratio; ++s) { any |= s_listed[s * nk + j]; all &= s_listed[s * nk + j]; }
    if ((all & 2u) || !(any & 1u)) continue;                        // tall-full or not listed: the plane is not read
    for (int s = 0; s < ratio; ++s) {
      const uint32_t f = s_listed[s * nk + j];
      if (f == 1u) continue;                                        // listed as partial: the mask's own bits
      const uint32_t word = f == 3u ? 0xffffffffu : 0u;
      for (int x = 0; x < wpb; ++x) {
        uint32_t* dst = plane_bits + (static_cast<int64_t>(j) * wpb + x) * p_out.Sq + row0 + s * bq_in;
        for (int r = lane; r < bq_in; r += 32) dst[r] = word;
      }
    }
  }
}

}  // namespace

cudaError_t launch_classify(const ClassifyParams& p, cudaStream_t stream) {
  const int planes = p.Bu * p.Hu;
  const int chunks = (p.Sk + kStripBytes - 1) / kStripBytes;
  const long long n_strips = static_cast<long long>(planes) * (p.Sq / kCell) * chunks;
  static int sm_count = 0, cells_occ = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    int sms = 0, occ = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, classify_cells_kernel, kCellsThreads, 0);
    if (e != cudaSuccess) return e;
    cells_occ = occ > 0 ? occ : 1;
    sm_count = sms;
  }
  const long long warps_per_cta = kCellsThreads / 32;
  long long ctas = (n_strips + warps_per_cta - 1) / warps_per_cta;
  const long long resident = static_cast<long long>(sm_count) * cells_occ;
  if (ctas > resident) ctas = resident;      // persistent: each warp strides over the strips
  if (ctas < 1) ctas = 1;
  classify_cells_kernel<<<static_cast<unsigned>(ctas), kCellsThreads, 0, stream>>>(p, chunks, n_strips);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int n_rows = planes * (p.Sq / p.BQ);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(n_rows));
  cfg.blockDim = dim3(kListsThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, compact_lists_kernel, p, n_rows);
}

// p_out carries only the output pointers; its block sizes are set here so that build_lists sees one
// flag row per short block and one flag per kv block.
cudaError_t launch_merge_lists(const int32_t* full_ids_in, const int32_t* full_lens_in, const int32_t* part_ids_in,
                               const int32_t* part_lens_in, int planes, int nq_out, int nk, int ratio,
                               int bq_in, int bk, ClassifyParams p_out, cudaStream_t stream) {
  p_out.BQ = kCell * ratio;
  p_out.BK = kCell;
  p_out.Sk = kCell * nk;
  p_out.Sq = nq_out * ratio * bq_in;
  const size_t smem = static_cast<size_t>(ratio) * static_cast<size_t>(nk);
  merge_lists_kernel<<<static_cast<unsigned>(planes * nq_out), kListsThreads, smem, stream>>>(
      p_out, full_ids_in, full_lens_in, part_ids_in, part_lens_in, nq_out, nk, ratio, bq_in, bk);
  return cudaGetLastError();
}

}  // namespace sa

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the classifier entry point.
//
// sa_classify_mask() needs a caller-provided workspace for the cell flags that travel between its
// two kernels.  Some hosts have no way to provide one: a serving process whose device memory was
// carved up once at start-up and is fully committed (KV caches, weights), a plugin that runs inside
// another runtime's callback where calling the allocator is not permitted, a hard-latency loop in
// which an allocation (and the implicit synchronisation a cudaMalloc / cudaFree can bring) is not
// affordable.  For them the flags live in the fixed device array below: SA_STATIC_SCRATCH_BYTES
// bytes that every GPU which loads this library holds until the process exits.
//
// The array's name is only a host-side handle; the device address is looked up once per device
// with cudaGetSymbolAddress (with that device current) on the first call made on it.  That first
// call therefore does set-up work and should be made before any stream capture is started.
// Every call uses the same array: it keeps the flags of the previous call (every flag a call reads
// is written by that call first, so nothing needs clearing), and two calls whose kernels overlap on
// the GPU - different streams, or different host threads - race on it.  Serialise them.
static __device__ __align__(256) uint8_t g_static_scratch[SA_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
uint8_t* g_static_scratch_addr[kMaxDevices] = {};
}  // namespace

extern "C" int sa_classify_mask_static(const uint8_t* mask,
                                       int64_t stride_b, int64_t stride_h, int64_t stride_q, int64_t stride_k,
                                       int B, int H, int Sq, int Sk, int BLOCK_Q, int BLOCK_K,
                                       int32_t* full_ids, int32_t* full_lens,
                                       int32_t* part_ids, int32_t* part_lens,
                                       uint32_t* packed_bits, void* stream) {
  if (B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0) return SA_ERR_INVALID_ARGUMENT;
  int Bu = 1, Hu = 1;
  if (sa_unique_planes(B, H, stride_b, stride_h, &Bu, &Hu) != SA_OK) return SA_ERR_INVALID_ARGUMENT;
  const size_t need = sa_classify_workspace_bytes(Bu, Hu, Sq, Sk);
  if (need == 0) return SA_ERR_INVALID_ARGUMENT;
  if (need > SA_STATIC_SCRATCH_BYTES) return SA_ERR_WORKSPACE;    // mask too large for the fixed array
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SA_ERR_NO_DEVICE;
  if (g_static_scratch_addr[dev] == nullptr) {
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_static_scratch) != cudaSuccess || addr == nullptr) return SA_ERR_CUDA;
    g_static_scratch_addr[dev] = static_cast<uint8_t*>(addr);
  }
  return sa_classify_mask(mask, stride_b, stride_h, stride_q, stride_k, B, H, Sq, Sk, BLOCK_Q, BLOCK_K,
                          full_ids, full_lens, part_ids, part_lens, packed_bits,
                          g_static_scratch_addr[dev], SA_STATIC_SCRATCH_BYTES, stream);
}
