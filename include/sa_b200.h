/* C ABI of libsparseattn_b200.so -- the two-stage block-sparse attention forward
 * path of tomatillos/sparseattention on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and element strides; no
 * torch types cross this boundary.  The caller owns every buffer (inputs,
 * outputs, workspace).  All work is enqueued on the given CUDA stream of the
 * current device and the calls do not synchronise.  Return value: 0 on success,
 * a negative SA_ERR_* otherwise (nothing is launched on an argument error).
 * The library never falls back to the CPU.
 */
#ifndef SA_B200_H_
#define SA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SA_ABI_VERSION 5

/* status codes */
#define SA_OK                     0
#define SA_ERR_INVALID_ARGUMENT  -1   /* null pointer, non-positive size, block size not dividing S */
#define SA_ERR_UNSUPPORTED       -2   /* shape / dtype / layout outside the supported set */
#define SA_ERR_WORKSPACE         -3   /* workspace missing or too small */
#define SA_ERR_CUDA              -4   /* a CUDA runtime / driver call failed (launch error included) */
#define SA_ERR_NO_DEVICE         -5   /* no usable sm_100 device is current */

/* element types of Q, K, V, O */
#define SA_DTYPE_F32   0
#define SA_DTYPE_F16   1
#define SA_DTYPE_BF16  2

/* attention kernel selection */
#define SA_IMPL_AUTO     0   /* tcgen05 kernel when the call is inside its supported set, else the SIMT kernel */
#define SA_IMPL_SIMT     1   /* generic fp32-accumulate CUDA-core kernel (any dtype, any block size) */
#define SA_IMPL_TCGEN05  2   /* TMA + tcgen05/TMEM kernel; SA_ERR_UNSUPPORTED outside its set */

/* values written to *dev_status by the attention kernel (0 = no device-side problem) */
#define SA_DEV_OK             0
#define SA_DEV_WAIT_EXPIRED   1   /* a bounded mbarrier wait ran out; the output is not valid */
#define SA_DEV_BAD_INDEX      2   /* a kv-block id outside [0, Sk/BLOCK_K) was found in a list, or (generic
                                     kernel) a list length outside [0, Sk/BLOCK_K]; such entries are skipped */

int sa_abi_version(void);
const char* sa_status_str(int status);

/* Number of distinct mask planes of a [B,H,Sq,Sk] mask whose batch / head strides
 * may be 0 (an expanded, broadcast mask: sparse_attn_kernel.py:154).  The
 * classifier reads and lists each distinct plane once: outputs have leading dims
 * [*Bu, *Hu] with Bu = (stride_b == 0 ? 1 : B), Hu = (stride_h == 0 ? 1 : H). */
int sa_unique_planes(int B, int H, int64_t stride_b, int64_t stride_h, int* Bu, int* Hu);

/* Bytes of scratch sa_classify_mask needs for any BLOCK_Q, BLOCK_K: the words through which the warps
 * that stream the mask hand the tile flags of a query block to the warp that builds its lists, and a
 * few counters.  8-byte aligned device memory. */
size_t sa_classify_workspace_bytes(int Bu, int Hu, int Sq, int Sk);

/* What the caller knows about the contents of a classifier workspace. */
#define SA_WS_UNKNOWN  0   /* anything (fresh allocation): the call clears it on the stream first (one small memset) */
#define SA_WS_CLEAN    1   /* zero-filled by the caller, or last used by a sa_classify_mask call that has run
                              to completion: the kernel leaves the workspace zero-filled, so a workspace that
                              is kept between calls needs clearing only once */

/* Stage 1: block classifier.  Replaces compute_mask_kernel / _compute_mask_inner
 * (sparseattention/mask_utils.py:85-107, 47-82).
 *
 * mask: bool bytes [B,H,Sq,Sk] (non-zero = attend) with element strides; stride_k
 *   must be 1 and every row start 16-byte aligned (else SA_ERR_UNSUPPORTED: make it
 *   contiguous first).  Sq % BLOCK_Q == 0 and Sk % BLOCK_K == 0 as in
 *   mask_utils.py:89-90; BLOCK_Q and BLOCK_K multiples of 32, BLOCK_Q at most 1024.
 * full_ids, part_ids: int32 [Bu,Hu,Sq/BLOCK_Q,Sk/BLOCK_K] contiguous; ascending kv-block
 *   ids of the fully-unmasked / partially-masked tiles of each query block, tail -1
 *   (mask_utils.py:72-79; the reference leaves the tail uninitialised).
 * full_lens, part_lens: int32 [Bu,Hu,Sq/BLOCK_Q] contiguous (mask_utils.py:81-82).
 * packed_bits: optional uint32 [Bu,Hu,Sk/32,Sq]; bit j of word [.,.,c,r] = mask[.,.,r,32c+j].
 *   Stage 2's tcgen05 kernel stages partial tiles from this plane instead of the byte mask.
 * workspace: sa_classify_workspace_bytes() bytes of device memory; workspace_state: SA_WS_UNKNOWN or
 *   SA_WS_CLEAN.  Calls that may overlap on the GPU need a workspace each. */
int sa_classify_mask(const uint8_t* mask,
                     int64_t stride_b, int64_t stride_h, int64_t stride_q, int64_t stride_k,
                     int B, int H, int Sq, int Sk, int BLOCK_Q, int BLOCK_K,
                     int32_t* full_ids, int32_t* full_lens,
                     int32_t* part_ids, int32_t* part_lens,
                     uint32_t* packed_bits,
                     void* workspace, size_t workspace_bytes, int workspace_state,
                     void* stream);

/* No counterpart in the reference.  The same classification as sa_classify_mask() for hosts that
 * cannot hand over a workspace because they cannot allocate device memory where this is called
 * (memory fully committed at start-up, allocator off-limits inside a foreign runtime's callback,
 * latency budget with no room for an allocation).  The scratch is a fixed device array inside the
 * library, SA_STATIC_SCRATCH_BYTES long, resident on every GPU that loads the library; the call
 * allocates nothing.  Masks whose scratch need (sa_classify_workspace_bytes) exceeds it are refused
 * with SA_ERR_WORKSPACE.  The first call on a device looks the array's address up (set-up work: make
 * that call before starting any stream capture; the address stays valid for the lifetime of the
 * device's primary context).  All calls share the array, which each call finds and leaves zero-filled,
 * so calls that may overlap on the GPU must be serialised by the caller. */
#define SA_STATIC_SCRATCH_BYTES (1u << 20)
int sa_classify_mask_static(const uint8_t* mask,
                            int64_t stride_b, int64_t stride_h, int64_t stride_q, int64_t stride_k,
                            int B, int H, int Sq, int Sk, int BLOCK_Q, int BLOCK_K,
                            int32_t* full_ids, int32_t* full_lens,
                            int32_t* part_ids, int32_t* part_lens,
                            uint32_t* packed_bits, void* stream);

/* No counterpart in the reference.  Folds lists made for query blocks `ratio` times shorter than the
 * ones wanted into lists for the tall blocks: a kv block is full for a tall block when it is in the
 * full list of each of its `ratio` short blocks, partial when any of them lists it and it is not full.
 * This is how lists built at BLOCK_Q = 32 or 64 (the reference's test_attn.py:32 uses (32, 128)) are
 * brought to the 128-row tiles of the tcgen05 kernel; the packed bit plane masks the elements.
 * Inputs: int32 [planes, nq_in, nk] ids and [planes, nq_in] lengths, contiguous; ids[..., :len] are
 * read.  Outputs: [planes, nq_in / ratio, nk] ids (ascending, tails -1) and [planes, nq_in / ratio].
 * packed_bits: optional plane [planes, nk * BLOCK_K / 32, nq_in * BLOCK_Q_in] made from the mask
 *   (sa_classify_mask), modified in place: inside the tall partial tiles, rows of a short block that
 *   does not list the kv block become all False and rows of one that lists it as full all True, so
 *   that stage 2 computes what a walk over the short lists computes even when the caller has edited
 *   them (lists derived from the same mask leave the plane unchanged). */
int sa_merge_lists(const int32_t* full_ids_in, const int32_t* full_lens_in,
                   const int32_t* part_ids_in, const int32_t* part_lens_in,
                   int planes, int nq_in, int nk, int ratio, int BLOCK_Q_in, int BLOCK_K,
                   int32_t* full_ids_out, int32_t* full_lens_out,
                   int32_t* part_ids_out, int32_t* part_lens_out,
                   uint32_t* packed_bits, void* stream);

/* Whether SA_IMPL_AUTO would pick the tcgen05 kernel for this call (1) or the SIMT kernel (0). */
int sa_attn_uses_tcgen05(int dtype, int D, int BLOCK_Q, int BLOCK_K, int Sq, int Sk,
                         const void* q, const void* k, const void* v,
                         const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                         int has_packed_bits);

/* Bytes of scratch sa_attn_fwd can use (a counter from which the CTAs of the tcgen05 kernel draw their
 * (query block, batch, head) tiles, so that uneven lists do not leave SMs idle at the end). */
size_t sa_attn_workspace_bytes(void);

/* Stage 2: block-sparse attention forward.  Replaces sparse_attention /
 * sparse_attention_kernel / _sparse_inner (sparseattention/sparse_attn_kernel.py:149-185,
 * 72-146, 10-63): per query block, a mask-free loop over the full list, then a masked
 * loop over the partial list, online softmax in base 2 with fp32 state, O = acc / l.
 * Rows with no attended key produce 0 (the reference produces NaN; torch SDPA gives 0).
 *
 * q,o: [B,H,Sq,D]; k,v: [B,H,Sk,D]; *_strides: 4 element strides each (b,h,s,d).
 * mask: bool bytes [B,H,Sq,Sk] with 4 element strides (0 allowed); read by the SIMT kernel.
 * packed_bits: uint32 plane from sa_classify_mask with (b,h) strides in words, or NULL
 *   (required by the tcgen05 kernel).
 * full_ids/part_ids: int32 with 4 element strides (b,h,q,k); full_lens/part_lens: int32 with
 *   3 element strides (b,h,q).  Only ids[..., :len] is read; they are trusted like the
 *   reference trusts a caller-supplied MaskMetadata (sparse_attn_kernel.py:157-163).
 * scale_log2: softmax scale already multiplied by log2(e) (sparse_attn_kernel.py:152).
 * lse: optional float32 [B,H,Sq] contiguous (no counterpart in the reference, which lists it as future
 *   work for a backward pass): per query row, log(sum over attended keys of exp(q.k * scale)), natural
 *   log; -inf for a row with no attended key.
 * workspace: optional sa_attn_workspace_bytes() bytes of device memory, 4-byte aligned; the call clears
 *   it on the stream.  NULL (or too small): the tiles are dealt to the CTAs in a fixed round-robin order.
 *   Calls that may overlap on the GPU need a workspace each.
 * dev_status: optional device int32, set non-zero by the kernel on a device-side problem. */
int sa_attn_fwd(const void* q, const void* k, const void* v, void* o,
                const int64_t* q_strides, const int64_t* k_strides,
                const int64_t* v_strides, const int64_t* o_strides,
                int dtype, int B, int H, int Sq, int Sk, int D, int BLOCK_Q, int BLOCK_K,
                const uint8_t* mask, const int64_t* mask_strides,
                const uint32_t* packed_bits, int64_t bits_stride_b, int64_t bits_stride_h,
                const int32_t* full_ids, const int64_t* full_ids_strides,
                const int32_t* full_lens, const int64_t* full_lens_strides,
                const int32_t* part_ids, const int64_t* part_ids_strides,
                const int32_t* part_lens, const int64_t* part_lens_strides,
                float scale_log2, int impl, float* lse, void* workspace, size_t workspace_bytes,
                int32_t* dev_status, void* stream);

/* No counterpart in the reference (a decode kernel is future work there, README.md:61-65).  The same
 * operation as sa_attn_fwd for calls with few query blocks and long key sequences (decoding, short
 * chunks of queries against a long cache), where one CTA per (query block, batch, head) leaves most of
 * the GPU idle: the walk of every (query block, batch, head) over its two lists is cut into `splits`
 * contiguous ranges that run as work items of their own on the tcgen05 kernel and leave normalised
 * partial outputs and log-sum-exps in the workspace; a second kernel combines them
 * (o = sum_s w_s o_s / sum_s w_s, w_s = exp(lse_s - max lse)).  splits = 1 is sa_attn_fwd on the tcgen05
 * kernel.  Arguments as for sa_attn_fwd; the call must lie inside the tcgen05 kernel's set
 * (sa_attn_uses_tcgen05), else SA_ERR_UNSUPPORTED.  workspace: sa_attn_splitkv_workspace_bytes(...) bytes,
 * 128-byte aligned (SA_ERR_WORKSPACE otherwise); calls that may overlap on the GPU need one each. */
size_t sa_attn_splitkv_workspace_bytes(int dtype, int B, int H, int Sq, int D, int splits);
int sa_attn_fwd_splitkv(const void* q, const void* k, const void* v, void* o,
                        const int64_t* q_strides, const int64_t* k_strides,
                        const int64_t* v_strides, const int64_t* o_strides,
                        int dtype, int B, int H, int Sq, int Sk, int D, int BLOCK_Q, int BLOCK_K,
                        const uint8_t* mask, const int64_t* mask_strides,
                        const uint32_t* packed_bits, int64_t bits_stride_b, int64_t bits_stride_h,
                        const int32_t* full_ids, const int64_t* full_ids_strides,
                        const int32_t* full_lens, const int64_t* full_lens_strides,
                        const int32_t* part_ids, const int64_t* part_ids_strides,
                        const int32_t* part_lens, const int64_t* part_lens_strides,
                        float scale_log2, int splits, float* lse, void* workspace, size_t workspace_bytes,
                        int32_t* dev_status, void* stream);

/* No counterpart in the reference (its README lists a backward pass as future work, README.md:61-65).
 * kv-major lists from the query-major lists of sa_classify_mask: for every (plane, kv block) the
 * ascending query blocks that list it as full / as partial, tails -1.  Inputs: int32 [planes, nq, nk]
 * ids and [planes, nq] lengths, contiguous.  Outputs: [planes, nk, nq] ids and [planes, nk] lengths. */
int sa_transpose_lists(const int32_t* full_ids, const int32_t* full_lens,
                       const int32_t* part_ids, const int32_t* part_lens,
                       int planes, int nq, int nk,
                       int32_t* t_full_ids, int32_t* t_full_lens,
                       int32_t* t_part_ids, int32_t* t_part_lens, void* stream);

/* Bytes of scratch sa_attn_bwd needs (one float per query row). */
size_t sa_attn_bwd_workspace_bytes(int B, int H, int Sq);

/* No counterpart in the reference.  Gradients of sa_attn_fwd with respect to q, k and v over the same
 * lists: P is recomputed from lse (the forward's optional output; a row whose lse is -inf has no
 * gradient), dV = P^T dO, dS = P * (dO V^T - D), dQ = scale dS K, dK = scale dS^T Q, with
 * D = rowsum(dO * O) - d_lse.  Any of the three dtypes, D in {16, 32, 64, 128}, block sizes that are
 * multiples of 32; no atomics (the result does not depend on scheduling).  fp16 / bf16 with D = 64 or
 * 128, unit stride along D and 16-byte aligned rows in every tensor run on the tensor cores (fp32
 * accumulation, P and dS rounded to the input type like the forward's P); everything else on the CUDA
 * cores in fp32.
 * o, d_o: the forward's output and its incoming gradient, [B,H,Sq,D] with element strides; lse: float32
 *   [B,H,Sq] contiguous from the forward; d_lse: optional incoming gradient of lse, same layout, or NULL.
 * dq, dk, dv: outputs with element strides, dtype of q.
 * full_* / part_*: the query-major lists given to the forward; t_*: the kv-major lists of
 *   sa_transpose_lists, with element strides ([B,H,nk,nq] / [B,H,nk]; 0 strides for broadcast planes).
 * workspace: sa_attn_bwd_workspace_bytes() bytes, 4-byte aligned. */
int sa_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                const float* lse, const float* d_lse,
                void* dq, void* dk, void* dv,
                const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                const int64_t* o_strides, const int64_t* do_strides,
                const int64_t* dq_strides, const int64_t* dk_strides, const int64_t* dv_strides,
                int dtype, int B, int H, int Sq, int Sk, int D, int BLOCK_Q, int BLOCK_K,
                const uint8_t* mask, const int64_t* mask_strides,
                const int32_t* full_ids, const int64_t* full_ids_strides,
                const int32_t* full_lens, const int64_t* full_lens_strides,
                const int32_t* part_ids, const int64_t* part_ids_strides,
                const int32_t* part_lens, const int64_t* part_lens_strides,
                const int32_t* t_full_ids, const int64_t* t_full_ids_strides,
                const int32_t* t_full_lens, const int64_t* t_full_lens_strides,
                const int32_t* t_part_ids, const int64_t* t_part_ids_strides,
                const int32_t* t_part_lens, const int64_t* t_part_lens_strides,
                float scale_log2, void* workspace, size_t workspace_bytes,
                int32_t* dev_status, void* stream);

/* No counterpart in the reference.  Self-test of the bounded device-side wait that every mbarrier wait of
 * the attention kernel goes through: launches one small CTA that waits on a barrier nothing will ever
 * arrive on, with the given limit (nanoseconds, at most 100 ms).  The wait must run out, the kernel must
 * return by itself and *dev_status must read SA_DEV_WAIT_EXPIRED; *waited_ns (optional, device memory)
 * receives how long the wait lasted. */
int sa_selftest_bounded_wait(uint64_t limit_ns, int32_t* dev_status, uint64_t* waited_ns, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SA_B200_H_ */
