/* CPU restatement of the reference block classifier, in C (test infrastructure).
 *
 * Same algorithm as sparseattention/mask_utils.py:14-44 (compute_mask_slow) and
 * the Triton kernel at mask_utils.py:47-82: count the True bytes of every
 * BLOCK_Q x BLOCK_K tile, append the kv-block id to the full list when the count
 * equals BLOCK_Q*BLOCK_K, to the partial list when it is positive, skip it when
 * zero; ids ascending; list tails are filled with -1 (the reference leaves them
 * uninitialised, mask_utils.py:91-94).
 *
 * Used by the tests as a second, independent checker and by the benchmark's CPU
 * baseline (one OpenMP thread per (slice, query block) row).  Never linked into
 * the shipped library.
 */
#include <stdint.h>
#include <stddef.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int sa_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* mask: n_slices contiguous [Sq, Sk] byte planes (non-zero byte = attend).
 * full_ids / part_ids: int32 [n_slices, Sq/BQ, Sk/BK]; lens: int32 [n_slices, Sq/BQ]. */
int sa_oracle_classify(const uint8_t* mask, int64_t n_slices, int64_t Sq, int64_t Sk,
                       int64_t BQ, int64_t BK,
                       int32_t* full_ids, int32_t* full_lens,
                       int32_t* part_ids, int32_t* part_lens) {
  if (BQ <= 0 || BK <= 0 || Sq % BQ || Sk % BK) return -1;   /* mask_utils.py:19-20 */
  const int64_t nq = Sq / BQ, nk = Sk / BK;
  const int64_t rows = n_slices * nq;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t s = r / nq, i = r % nq;
    const uint8_t* base = mask + (s * Sq + i * BQ) * Sk;
    int32_t* fo = full_ids + r * nk;
    int32_t* po = part_ids + r * nk;
    int32_t nf = 0, np = 0;
    for (int64_t j = 0; j < nk; ++j) {                        /* mask_utils.py:31 */
      int64_t count = 0;
      for (int64_t y = 0; y < BQ; ++y) {
        const uint8_t* row = base + y * Sk + j * BK;
        int64_t c = 0;
        for (int64_t x = 0; x < BK; ++x) c += row[x] != 0;
        count += c;
      }
      if (count == BQ * BK) fo[nf++] = (int32_t)j;            /* mask_utils.py:34-36 */
      else if (count > 0)   po[np++] = (int32_t)j;            /* mask_utils.py:37-39 */
    }
    for (int64_t t = nf; t < nk; ++t) fo[t] = -1;
    for (int64_t t = np; t < nk; ++t) po[t] = -1;
    full_lens[r] = nf;                                        /* mask_utils.py:40-41 */
    part_lens[r] = np;
  }
  return 0;
}
