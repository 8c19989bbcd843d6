// Stage 1: block classifier for a dense boolean attention mask (HBM-bound).
//
// Replaces sparseattention/mask_utils.py:47-107 (_compute_mask_inner + its launcher).
// The reference walks the kv blocks of one query block serially in one program and
// re-reads an expanded mask once per head; here every distinct mask byte is read
// exactly once with 16-byte loads, by ONE kernel:
//
//   streaming   one warp per strip of 32 rows x 512 columns: each lane streams 32 rows of 16 bytes,
//               reduces them to "any / all" flags of the 32x32 cells (a lane pair per cell) and,
//               optionally, emits the packed bit-plane stage 2 reads.  The grid is SMs x resident CTAs
//               (four of 256 threads per SM); every warp strides over the strips.
//   flags       the 16 cells of a strip travel as one 64-bit atomic OR into a word per (plane, query
//               block, strip column): 16 "any" bits, 16 "not all" bits and one arrival bit per cell
//               row of the query block.  The warp whose OR completes a word counts it on the query
//               block; the warp that counts the last word of a query block has, by then, every flag
//               of that block in front of it.
//   lists       that warp folds the flags of each BLOCK_Q x BLOCK_K tile, ballots the full / partial
//               predicates and writes the ascending id lists by popcount prefixes (order of
//               mask_utils.py:66-79), tails filled with -1, and puts the words and the counter back
//               to zero (it fetches the words with atomic exchanges that leave zero behind).  List building thus overlaps the streaming of the rest of the mask; only the
//               last query block's lists are built after the last byte has arrived.
//
// Scratch: the words and counters (sa_classify_workspace_bytes).  They must be zero when the kernel
// starts and are zero again when it ends.
#include <atomic>
#include <mutex>

#include "sa_common.cuh"

namespace sa {
namespace {

__device__ __forceinline__ uint4 ld_stream_16(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(selector));
  return r;
}

// 16 mask bytes, each 0 or 1 -> 16 bits in the low half of the result (bit i = byte i); the upper half
// is not meaningful.  A multiply gathers the four low bits of a word's bytes into its top byte (into the
// low nibble with one constant, the high nibble with the other), so two words share a byte.
__device__ __forceinline__ uint32_t bits_of_01(const uint4& v) {
  const uint32_t a = (v.x * 0x01020408u) | (v.y * 0x10204080u);
  const uint32_t b = (v.z * 0x01020408u) | (v.w * 0x10204080u);
  return prmt(a, b, 0x0073u);            // byte 0 <- top byte of a, byte 1 <- top byte of b
}

// Any non-zero byte -> 1 (torch bool storage is 0 / 1 already; a mask viewed from other bytes may not be).
__device__ __forceinline__ uint32_t to_01(uint32_t w) {
  return ((((w & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w) >> 7) & 0x01010101u;
}

constexpr int kCellsThreads = 256;
constexpr int kWarpsPerCta = kCellsThreads / 32;
constexpr int kCellsPerStrip = kStripBytes / kCell;       // 16

// The lists of one (plane, query block) from its flag words, by one warp.  words[c]: bits 0-15 "any
// True" and bits 16-31 "not all True" of the 16 cell columns of strip column c, ORed over the cell
// rows of the query block.  The words are fetched with an atomic exchange that leaves zero behind
// (every atomic on a word is performed where the word lives, so the exchange returns every
// contribution that was acknowledged before it); 32 tiles per pass, one per lane.
__device__ __forceinline__ void build_lists_warp(const ClassifyParams& p, unsigned long long* words,
                                                 int chunks_per_row, int row) {
  const int lane = threadIdx.x & 31;
  const int nk = p.Sk / p.BK;
  const int rk = p.BK / kCell;
  int32_t* f_out = p.full_ids + static_cast<int64_t>(row) * nk;
  int32_t* p_out = p.part_ids + static_cast<int64_t>(row) * nk;
  const uint32_t lt_mask = (1u << lane) - 1u;
  int nf = 0, np = 0;
  auto emit = [&](int j, bool live, bool any, bool all) {
    const bool is_full = live && all;                                  // count == BQ*BK  (mask_utils.py:72)
    const bool is_part = live && !all && any;                          // 0 < count       (mask_utils.py:76)
    const uint32_t bf = __ballot_sync(0xffffffffu, is_full);
    const uint32_t bp = __ballot_sync(0xffffffffu, is_part);
    if (is_full) f_out[nf + __popc(bf & lt_mask)] = j;
    if (is_part) p_out[np + __popc(bp & lt_mask)] = j;
    nf += __popc(bf);
    np += __popc(bp);
  };
  if (chunks_per_row <= 32 || (32 * kCellsPerStrip) % rk == 0) {
    // 32 strip columns (512 cell columns) at a time, lane l holding word w0 + l: no tile straddles two
    // such groups
    for (int w0 = 0; w0 < chunks_per_row; w0 += 32) {
      const uint32_t mine = (w0 + lane < chunks_per_row)
          ? static_cast<uint32_t>(atomicExch(words + w0 + lane, 0ull)) : 0u;
      const int cell_end = min((w0 + 32) * kCellsPerStrip, p.Sk / kCell);
      for (int j0 = w0 * kCellsPerStrip / rk; j0 * rk < cell_end; j0 += 32) {
        const int j = j0 + lane;
        bool any = false, all = true;
        for (int x = 0; x < rk; ++x) {
          const int cc = j * rk + x;                                   // cell column
          const uint32_t w = __shfl_sync(0xffffffffu, mine, ((cc >> 4) - w0) & 31);
          any = any || ((w >> (cc & 15)) & 1u);
          all = all && !((w >> (16 + (cc & 15))) & 1u);
        }
        emit(j, j * rk < cell_end && j < nk, any, all);
      }
    }
  } else {
    // long rows with a BLOCK_K whose tiles can straddle a group of 32 words: every lane reads the words
    // of its tile itself (an atomic OR of nothing returns the word), and the words are cleared afterwards
    for (int j0 = 0; j0 < nk; j0 += 32) {
      const int j = j0 + lane;
      bool any = false, all = true;
      if (j < nk) {
        for (int x = 0; x < rk; ++x) {
          const int cc = j * rk + x;
          const uint32_t w = static_cast<uint32_t>(atomicOr(words + (cc >> 4), 0ull));
          any = any || ((w >> (cc & 15)) & 1u);
          all = all && !((w >> (16 + (cc & 15))) & 1u);
        }
      }
      emit(j, j < nk, any, all);
    }
    __syncwarp();
    for (int c = lane; c < chunks_per_row; c += 32) atomicExch(words + c, 0ull);
  }
  for (int t = nf + lane; t < nk; t += 32) f_out[t] = -1;
  for (int t = np + lane; t < nk; t += 32) p_out[t] = -1;
  if (lane == 0) {
    p.full_lens[row] = nf;                                             // mask_utils.py:81
    p.part_lens[row] = np;                                             // mask_utils.py:82
  }
}

// 32 rows x 16 bytes of one lane -> the lane's AND / OR accumulators over the rows (16 bits each) and,
// exchanged with the neighbour lane, the 32-bit row words of the lane pair's cell: even lanes keep rows
// 0..15 of the cell, odd lanes rows 16..31.  kNormalise: bytes other than 0 / 1 may occur.
template <bool kNormalise>
__device__ __forceinline__ void reduce_strip(const uint8_t* src, int64_t stride_q, bool active, int odd,
                                             uint32_t& and_acc, uint32_t& or_acc, uint32_t& raw_or,
                                             uint32_t (&keep)[16]) {
  const uint32_t selector = odd ? 0x1054u : 0x5410u;       // (mine, other) -> columns in ascending order
  and_acc = 0xffffu;
  or_acc = 0u;
  raw_or = 0u;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 v[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      v[r] = active ? ld_stream_16(src + static_cast<int64_t>(g * 8 + r) * stride_q) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int row = g * 8 + r;
      if (kNormalise) {
        v[r].x = to_01(v[r].x); v[r].y = to_01(v[r].y); v[r].z = to_01(v[r].z); v[r].w = to_01(v[r].w);
      } else {
        raw_or |= v[r].x | v[r].y;
        raw_or |= v[r].z | v[r].w;
      }
      const uint32_t hb = bits_of_01(v[r]);
      and_acc &= hb;
      or_acc |= hb;
      const uint32_t other = __shfl_xor_sync(0xffffffffu, hb, 1);
      const uint32_t word = prmt(hb, other, selector);
      if ((row >> 4) == 0) { if (!odd) keep[row & 15] = word; }
      else                 { if (odd)  keep[row & 15] = word; }
    }
  }
  and_acc &= 0xffffu;
  or_acc &= 0xffffu;
}

__global__ void __launch_bounds__(kCellsThreads, 4)
classify_kernel(const ClassifyParams p, const int chunks_per_row, const long long n_strips) {
  const int lane = threadIdx.x & 31;
  const int row_cells = p.Sq / kCell;
  const int col_cells = p.Sk / kCell;
  const int rq = p.BQ / kCell, nq = p.Sq / p.BQ;
  const int odd = lane & 1;
  const unsigned long long done_all = rq >= 32 ? 0xffffffffull : ((1ull << rq) - 1ull);
  const long long n_warps = (static_cast<long long>(gridDim.x) * kCellsThreads) >> 5;

  for (long long strip = (static_cast<long long>(blockIdx.x) * kCellsThreads + threadIdx.x) >> 5; strip < n_strips;
       strip += n_warps) {
    const int chunk = static_cast<int>(strip % chunks_per_row);
    const long long t = strip / chunks_per_row;
    const int rc = static_cast<int>(t % row_cells);
    const int plane = static_cast<int>(t / row_cells);
    const int b = plane / p.Hu, h = plane % p.Hu;
    const int col = chunk * kStripBytes + lane * 16;
    const bool active = col < p.Sk;
    const uint8_t* src = p.mask + b * p.stride_b + h * p.stride_h +
                         static_cast<int64_t>(rc) * kCell * p.stride_q + col;

    uint32_t and_acc, or_acc, raw_or;
    uint32_t keep[16];
    reduce_strip<false>(src, p.stride_q, active, odd, and_acc, or_acc, raw_or, keep);
    if (__any_sync(0xffffffffu, (raw_or & 0xfefefefeu) != 0u))          // bytes other than 0 / 1: once more, normalised
      reduce_strip<true>(src, p.stride_q, active, odd, and_acc, or_acc, raw_or, keep);
    const uint32_t and_all = and_acc & __shfl_xor_sync(0xffffffffu, and_acc, 1);
    const uint32_t or_any = or_acc | __shfl_xor_sync(0xffffffffu, or_acc, 1);
    // cell c of the strip is owned by lanes 2c and 2c+1: bring its flags to lane c and ballot
    const int src_lane = (lane & 15) * 2;
    const bool any_c = __shfl_sync(0xffffffffu, or_any != 0u ? 1 : 0, src_lane) != 0;
    const bool all_c = __shfl_sync(0xffffffffu, and_all == 0xffffu ? 1 : 0, src_lane) != 0;
    const uint32_t any16 = __ballot_sync(0xffffffffu, any_c) & 0xffffu;
    const uint32_t notall16 = __ballot_sync(0xffffffffu, !all_c) & 0xffffu;

    // One 64-bit atomic carries the strip's flags and its arrival.  Everything the list builder needs
    // travels inside atomics, each issued after the previous one's value has come back: a strip's OR,
    // then (by the warp whose OR completed the word) the count on the query block, then (by the warp
    // that counted the last word) the exchanges that fetch the words.  All of them are performed at the
    // one place where their address lives, so an exchange returns every OR that was acknowledged before
    // the count that led to it; no other memory is handed between warps, and no fence is needed.
    const int qblk = rc / rq;
    const int64_t qrow = static_cast<int64_t>(plane) * nq + qblk;
    unsigned long long* words = p.words + qrow * chunks_per_row;
    int build = 0;
    if (lane == 0) {
      const unsigned long long mine = static_cast<unsigned long long>(any16) |
                                      (static_cast<unsigned long long>(notall16) << 16) |
                                      (1ull << (32 + (rc % rq)));
      const unsigned long long old = atomicOr(words + chunk, mine);
      if ((((old | mine) >> 32) & 0xffffffffull) == done_all) {
        const unsigned int seen = atomicAdd(p.row_counters + qrow, 1u);
        build = seen == static_cast<unsigned int>(chunks_per_row) - 1u;
      }
    }
    build = __shfl_sync(0xffffffffu, build, 0);
    if (build) {
      build_lists_warp(p, words, chunks_per_row, static_cast<int>(qrow));   // leaves the words zero
      if (lane == 0) atomicExch(p.row_counters + qrow, 0u);
    }
    if (active && p.bits != nullptr) {
      const int kb = chunk * kCellsPerStrip + (lane >> 1);
      uint4* dst = reinterpret_cast<uint4*>(
          p.bits + (static_cast<int64_t>(plane) * col_cells + kb) * p.Sq + rc * kCell + odd * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        dst[i] = make_uint4(keep[4 * i], keep[4 * i + 1], keep[4 * i + 2], keep[4 * i + 3]);
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

size_t classify_workspace_layout(int planes, int nq, int chunks, size_t* off_rows, size_t* off_words) {
  const size_t rows = static_cast<size_t>(planes) * nq;
  const size_t o_rows = 0;
  const size_t o_words = (o_rows + 4 * rows + 7) & ~static_cast<size_t>(7);
  if (off_rows != nullptr) *off_rows = o_rows;
  if (off_words != nullptr) *off_words = o_words;
  return o_words + 8 * rows * static_cast<size_t>(chunks);
}

cudaError_t launch_classify(ClassifyParams p, void* workspace, bool clear_first, cudaStream_t stream) {
  const int planes = p.Bu * p.Hu;
  const int chunks = (p.Sk + kStripBytes - 1) / kStripBytes;
  const int nq = p.Sq / p.BQ;
  const long long n_strips = static_cast<long long>(planes) * (p.Sq / kCell) * chunks;
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return cudaErrorInvalidDevice;
  static std::once_flag once[kMaxDevices];
  static int occupancy[kMaxDevices];
  std::call_once(once[info->ordinal], [&] {
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, classify_kernel, kCellsThreads, 0) != cudaSuccess) occ = 0;
    occupancy[info->ordinal] = occ > 0 ? occ : 1;
  });
  size_t off_rows = 0, off_words = 0;
  const size_t bytes = classify_workspace_layout(planes, nq, chunks, &off_rows, &off_words);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.row_counters = reinterpret_cast<unsigned int*>(ws + off_rows);
  p.words = reinterpret_cast<unsigned long long*>(ws + off_words);
  if (clear_first) {
    cudaError_t e = cudaMemsetAsync(ws, 0, bytes, stream);
    if (e != cudaSuccess) return e;
  }
  long long ctas = (n_strips + kWarpsPerCta - 1) / kWarpsPerCta;
  const long long resident = static_cast<long long>(info->sm_count) * occupancy[info->ordinal];
  if (ctas > resident) ctas = resident;      // persistent: each warp strides over the strips
  if (ctas < 1) ctas = 1;
  classify_kernel<<<static_cast<unsigned>(ctas), kCellsThreads, 0, stream>>>(p, chunks, n_strips);
  return cudaGetLastError();
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
// sa_classify_mask() needs a caller-provided workspace for the flag words and counters through which
// the warps of its kernel hand the tile flags to the warp that builds a query block's lists.  Some
// hosts have no way to provide one: a serving process whose device memory was carved up once at
// start-up and is fully committed (KV caches, weights), a plugin that runs inside another runtime's
// callback where calling the allocator is not permitted, a hard-latency loop in which an allocation
// (and the implicit synchronisation a cudaMalloc / cudaFree can bring) is not affordable.  For them
// the scratch lives in the fixed device array below: SA_STATIC_SCRATCH_BYTES bytes that every GPU
// which loads this library holds until the process exits.
//
// The array's name is only a host-side handle; the device address is looked up once per device
// with cudaGetSymbolAddress (with that device current) on the first call made on it.  That first
// call therefore does set-up work and should be made before any stream capture is started.  The
// cached address is valid for the lifetime of the device's primary context.
// Every call uses the same array.  The kernel needs it zero-filled and leaves it zero-filled (the
// array starts out as zeros, and each word is put back to zero by the warp that consumed it), so
// nothing is cleared between calls; two calls whose kernels overlap on the GPU - different streams,
// or different host threads - race on it.  Serialise them.
static __device__ __align__(256) uint8_t g_static_scratch[SA_STATIC_SCRATCH_BYTES];

namespace {
std::atomic<uint8_t*> g_static_scratch_addr[sa::kMaxDevices];
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
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= sa::kMaxDevices) return SA_ERR_NO_DEVICE;
  uint8_t* scratch = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_static_scratch) != cudaSuccess || addr == nullptr) return SA_ERR_CUDA;
    scratch = static_cast<uint8_t*>(addr);
    g_static_scratch_addr[dev].store(scratch, std::memory_order_release);   // every thread finds the same value
  }
  return sa_classify_mask(mask, stride_b, stride_h, stride_q, stride_k, B, H, Sq, Sk, BLOCK_Q, BLOCK_K,
                          full_ids, full_lens, part_ids, part_lens, packed_bits,
                          scratch, SA_STATIC_SCRATCH_BYTES, SA_WS_CLEAN, stream);
}
