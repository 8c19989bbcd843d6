// extern "C" entry points declared in include/sa_b200.h: argument validation and dispatch.
#include <cstring>
#include <mutex>

#include "sa_common.cuh"

namespace sa {

const DeviceInfo* current_device_info() {
  static std::once_flag once[kMaxDevices];
  static DeviceInfo info[kMaxDevices];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::call_once(once[dev], [dev] {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 0;
    info[dev].ordinal = dev;
    info[dev].sm_count = sms;
  });
  return info[dev].sm_count > 0 ? &info[dev] : nullptr;
}

}  // namespace sa

namespace {

bool positive(int x) { return x > 0; }

void copy_n(int64_t* dst, const int64_t* src, int n) {
  for (int i = 0; i < n; ++i) dst[i] = src[i];
}

}  // namespace

extern "C" {

int sa_abi_version(void) { return SA_ABI_VERSION; }

const char* sa_status_str(int status) {
  switch (status) {
    case SA_OK: return "ok";
    case SA_ERR_INVALID_ARGUMENT: return "invalid argument";
    case SA_ERR_UNSUPPORTED: return "unsupported shape, dtype or layout";
    case SA_ERR_WORKSPACE: return "workspace missing or too small";
    case SA_ERR_CUDA: return "CUDA call failed";
    case SA_ERR_NO_DEVICE: return "no usable device";
    default: return "unknown status";
  }
}

int sa_unique_planes(int B, int H, int64_t stride_b, int64_t stride_h, int* Bu, int* Hu) {
  if (!positive(B) || !positive(H) || Bu == nullptr || Hu == nullptr) return SA_ERR_INVALID_ARGUMENT;
  *Bu = (stride_b == 0) ? 1 : B;
  *Hu = (stride_h == 0) ? 1 : H;
  return SA_OK;
}

size_t sa_classify_workspace_bytes(int Bu, int Hu, int Sq, int Sk) {
  if (!positive(Bu) || !positive(Hu) || !positive(Sq) || !positive(Sk)) return 0;
  if (static_cast<long long>(Bu) * Hu > 0x7fffffffLL) return 0;
  // sized for the shortest query blocks (32 rows), whatever BLOCK_Q a call then uses
  const int chunks = (Sk + sa::kStripBytes - 1) / sa::kStripBytes;
  const size_t bytes = sa::classify_workspace_layout(Bu * Hu, (Sq + sa::kCell - 1) / sa::kCell, chunks, nullptr, nullptr);
  return (bytes + 255) & ~static_cast<size_t>(255);
}

int sa_classify_mask(const uint8_t* mask,
                     int64_t stride_b, int64_t stride_h, int64_t stride_q, int64_t stride_k,
                     int B, int H, int Sq, int Sk, int BLOCK_Q, int BLOCK_K,
                     int32_t* full_ids, int32_t* full_lens,
                     int32_t* part_ids, int32_t* part_lens,
                     uint32_t* packed_bits,
                     void* workspace, size_t workspace_bytes, int workspace_state,
                     void* stream) {
  if (mask == nullptr || full_ids == nullptr || full_lens == nullptr || part_ids == nullptr || part_lens == nullptr)
    return SA_ERR_INVALID_ARGUMENT;
  if (!positive(B) || !positive(H) || !positive(Sq) || !positive(Sk) || !positive(BLOCK_Q) || !positive(BLOCK_K))
    return SA_ERR_INVALID_ARGUMENT;
  if (Sq % BLOCK_Q != 0 || Sk % BLOCK_K != 0) return SA_ERR_INVALID_ARGUMENT;        // mask_utils.py:89-90
  if (BLOCK_Q % sa::kCell != 0 || BLOCK_K % sa::kCell != 0) return SA_ERR_UNSUPPORTED;
  if (BLOCK_Q > 32 * sa::kCell) return SA_ERR_UNSUPPORTED;       // one arrival bit per 32-row slice of a query block
  if (workspace_state != SA_WS_UNKNOWN && workspace_state != SA_WS_CLEAN) return SA_ERR_INVALID_ARGUMENT;
  if (stride_k != 1 || stride_q < Sk || stride_q % 16 != 0 || stride_b % 16 != 0 || stride_h % 16 != 0 ||
      stride_b < 0 || stride_h < 0 || reinterpret_cast<uintptr_t>(mask) % 16 != 0)
    return SA_ERR_UNSUPPORTED;
  if (packed_bits != nullptr && reinterpret_cast<uintptr_t>(packed_bits) % 16 != 0) return SA_ERR_UNSUPPORTED;
  int Bu = 1, Hu = 1;
  sa_unique_planes(B, H, stride_b, stride_h, &Bu, &Hu);
  const size_t need = sa_classify_workspace_bytes(Bu, Hu, Sq, Sk);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 8 != 0)
    return SA_ERR_WORKSPACE;
  if (static_cast<long long>(Bu) * Hu * (Sq / BLOCK_Q) > 0x7fffffffLL) return SA_ERR_UNSUPPORTED;

  sa::ClassifyParams p = {};
  p.mask = mask;
  p.stride_b = stride_b; p.stride_h = stride_h; p.stride_q = stride_q;
  p.Bu = Bu; p.Hu = Hu; p.Sq = Sq; p.Sk = Sk; p.BQ = BLOCK_Q; p.BK = BLOCK_K;
  p.bits = packed_bits;
  p.full_ids = full_ids; p.full_lens = full_lens; p.part_ids = part_ids; p.part_lens = part_lens;
  return sa::launch_classify(p, workspace, workspace_state == SA_WS_UNKNOWN, static_cast<cudaStream_t>(stream)) ==
                 cudaSuccess
             ? SA_OK : SA_ERR_CUDA;
}

int sa_merge_lists(const int32_t* full_ids_in, const int32_t* full_lens_in,
                   const int32_t* part_ids_in, const int32_t* part_lens_in,
                   int planes, int nq_in, int nk, int ratio, int BLOCK_Q_in, int BLOCK_K,
                   int32_t* full_ids_out, int32_t* full_lens_out,
                   int32_t* part_ids_out, int32_t* part_lens_out,
                   uint32_t* packed_bits, void* stream) {
  if (full_ids_in == nullptr || full_lens_in == nullptr || part_ids_in == nullptr || part_lens_in == nullptr ||
      full_ids_out == nullptr || full_lens_out == nullptr || part_ids_out == nullptr || part_lens_out == nullptr)
    return SA_ERR_INVALID_ARGUMENT;
  if (!positive(planes) || !positive(nq_in) || !positive(nk) || !positive(ratio) || nq_in % ratio != 0 ||
      !positive(BLOCK_Q_in) || !positive(BLOCK_K))
    return SA_ERR_INVALID_ARGUMENT;
  if (BLOCK_Q_in % sa::kCell != 0 || BLOCK_K % sa::kCell != 0) return SA_ERR_UNSUPPORTED;
  if (static_cast<size_t>(ratio) * static_cast<size_t>(nk) > 40u * 1024u) return SA_ERR_UNSUPPORTED;
  if (static_cast<long long>(planes) * (nq_in / ratio) > 0x7fffffffLL) return SA_ERR_UNSUPPORTED;
  sa::ClassifyParams p = {};
  p.full_ids = full_ids_out; p.full_lens = full_lens_out; p.part_ids = part_ids_out; p.part_lens = part_lens_out;
  p.bits = packed_bits;
  return sa::launch_merge_lists(full_ids_in, full_lens_in, part_ids_in, part_lens_in, planes, nq_in / ratio, nk,
                                ratio, BLOCK_Q_in, BLOCK_K, p, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? SA_OK : SA_ERR_CUDA;
}

static int fill_attn_params(sa::AttnParams& p,
                            const void* q, const void* k, const void* v, void* o,
                            const int64_t* q_strides, const int64_t* k_strides,
                            const int64_t* v_strides, const int64_t* o_strides,
                            int dtype, int B, int H, int Sq, int Sk, int D, int BLOCK_Q, int BLOCK_K) {
  if (q == nullptr || k == nullptr || v == nullptr || q_strides == nullptr || k_strides == nullptr ||
      v_strides == nullptr)
    return SA_ERR_INVALID_ARGUMENT;
  if (!positive(B) || !positive(H) || !positive(Sq) || !positive(Sk) || !positive(D) || !positive(BLOCK_Q) ||
      !positive(BLOCK_K))
    return SA_ERR_INVALID_ARGUMENT;
  if (Sq % BLOCK_Q != 0 || Sk % BLOCK_K != 0) return SA_ERR_INVALID_ARGUMENT;
  if (dtype != SA_DTYPE_F32 && dtype != SA_DTYPE_F16 && dtype != SA_DTYPE_BF16) return SA_ERR_UNSUPPORTED;
  std::memset(&p, 0, sizeof(p));
  p.q = q; p.k = k; p.v = v; p.o = o;
  copy_n(p.qs, q_strides, 4); copy_n(p.ks, k_strides, 4); copy_n(p.vs, v_strides, 4);
  if (o_strides != nullptr) copy_n(p.os, o_strides, 4);
  p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk; p.D = D; p.BQ = BLOCK_Q; p.BK = BLOCK_K; p.dtype = dtype;
  return SA_OK;
}

int sa_attn_uses_tcgen05(int dtype, int D, int BLOCK_Q, int BLOCK_K, int Sq, int Sk,
                         const void* q, const void* k, const void* v,
                         const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                         int has_packed_bits) {
  sa::AttnParams p;
  if (fill_attn_params(p, q, k, v, nullptr, q_strides, k_strides, v_strides, nullptr, dtype, 1, 1, Sq, Sk, D,
                       BLOCK_Q, BLOCK_K) != SA_OK)
    return 0;
  // output layout and bit-plane alignment are checked at launch; assume a fresh contiguous output here
  static const uint32_t aligned_dummy[4] __attribute__((aligned(16))) = {0, 0, 0, 0};
  p.bits = has_packed_bits ? aligned_dummy : nullptr;
  p.o = const_cast<uint32_t*>(aligned_dummy);
  p.os[3] = 1; p.os[2] = D; p.os[1] = static_cast<int64_t>(D) * Sq; p.os[0] = p.os[1];
  p.scale_log2 = 1.f;
  return sa::attn_tc_supported(p);
}

size_t sa_attn_workspace_bytes(void) { return 16; }

namespace {

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// workspace of a split walk: the tile counter, the partial log-sum-exps, the partial outputs
struct SplitLayout {
  size_t off_lse, off_o, total;
};
SplitLayout split_layout(int dtype, int B, int H, int Sq, int D, int splits) {
  SplitLayout l;
  const size_t rows = static_cast<size_t>(splits) * B * H * Sq;
  l.off_lse = 16;
  l.off_o = align_up(l.off_lse + rows * sizeof(float), 128);
  l.total = l.off_o + rows * D * (dtype == SA_DTYPE_F32 ? 4 : 2);
  return l;
}

int attn_fwd_common(const void* q, const void* k, const void* v, void* o,
                const int64_t* q_strides, const int64_t* k_strides,
                const int64_t* v_strides, const int64_t* o_strides,
                int dtype, int B, int H, int Sq, int Sk, int D, int BLOCK_Q, int BLOCK_K,
                const uint8_t* mask, const int64_t* mask_strides,
                const uint32_t* packed_bits, int64_t bits_stride_b, int64_t bits_stride_h,
                const int32_t* full_ids, const int64_t* full_ids_strides,
                const int32_t* full_lens, const int64_t* full_lens_strides,
                const int32_t* part_ids, const int64_t* part_ids_strides,
                const int32_t* part_lens, const int64_t* part_lens_strides,
                float scale_log2, int impl, int splits, float* lse, void* workspace, size_t workspace_bytes,
                int32_t* dev_status, void* stream) {
  sa::AttnParams p;
  if (o == nullptr || o_strides == nullptr) return SA_ERR_INVALID_ARGUMENT;
  int rc = fill_attn_params(p, q, k, v, o, q_strides, k_strides, v_strides, o_strides, dtype, B, H, Sq, Sk, D,
                            BLOCK_Q, BLOCK_K);
  if (rc != SA_OK) return rc;
  if (full_ids == nullptr || full_lens == nullptr || part_ids == nullptr || part_lens == nullptr ||
      full_ids_strides == nullptr || full_lens_strides == nullptr || part_ids_strides == nullptr ||
      part_lens_strides == nullptr)
    return SA_ERR_INVALID_ARGUMENT;
  if (impl != SA_IMPL_AUTO && impl != SA_IMPL_SIMT && impl != SA_IMPL_TCGEN05) return SA_ERR_INVALID_ARGUMENT;
  p.mask = mask;
  if (mask_strides != nullptr) copy_n(p.ms, mask_strides, 4);
  p.bits = packed_bits; p.bits_sb = bits_stride_b; p.bits_sh = bits_stride_h;
  p.full_ids = full_ids; copy_n(p.fis, full_ids_strides, 4);
  p.full_lens = full_lens; copy_n(p.fls, full_lens_strides, 3);
  p.part_ids = part_ids; copy_n(p.pis, part_ids_strides, 4);
  p.part_lens = part_lens; copy_n(p.pls, part_lens_strides, 3);
  p.scale_log2 = scale_log2;
  p.lse = lse;
  p.dev_status = dev_status;
  p.tile_counter = nullptr;
  p.splits = 1;
  if (workspace != nullptr && workspace_bytes >= sa_attn_workspace_bytes() &&
      reinterpret_cast<uintptr_t>(workspace) % 4 == 0)
    p.tile_counter = static_cast<int32_t*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  const bool tc_ok = sa::attn_tc_supported(p) != 0;
  if (splits > 1) {
    // The walk of every (query block, batch, head) over its lists is cut into `splits` ranges that run as
    // tiles of their own and leave normalised partial outputs and log-sum-exps in the workspace; a second
    // kernel combines them.  tcgen05 kernel only.
    if (!tc_ok) return SA_ERR_UNSUPPORTED;
    if (splits > 256 || static_cast<long long>(B) * splits > 0x7fffffLL) return SA_ERR_UNSUPPORTED;
    const SplitLayout lay = split_layout(dtype, B, H, Sq, D, splits);
    if (workspace == nullptr || workspace_bytes < lay.total || reinterpret_cast<uintptr_t>(workspace) % 128 != 0)
      return SA_ERR_WORKSPACE;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    sa::AttnParams ps = p;
    ps.splits = splits;
    ps.o = ws + lay.off_o;
    ps.os[3] = 1; ps.os[2] = D; ps.os[1] = static_cast<int64_t>(Sq) * D; ps.os[0] = ps.os[1] * H;
    ps.lse = reinterpret_cast<float*>(ws + lay.off_lse);
    const int rc2 = sa::launch_attn_tc(ps, s);
    if (rc2 != SA_OK) return rc2;
    return sa::launch_merge_splits(ps.o, ps.lse, splits, dtype, B, H, Sq, D, o, p.os, lse, s) == cudaSuccess
               ? SA_OK : SA_ERR_CUDA;
  }
  if (impl == SA_IMPL_TCGEN05 || (impl == SA_IMPL_AUTO && tc_ok)) return sa::launch_attn_tc(p, s);

  // generic kernel
  if (mask == nullptr || mask_strides == nullptr) return SA_ERR_INVALID_ARGUMENT;
  if (BLOCK_Q % 32 != 0 || BLOCK_K % 32 != 0) return SA_ERR_UNSUPPORTED;
  if (D != 16 && D != 32 && D != 64 && D != 128) return SA_ERR_UNSUPPORTED;
  return sa::launch_attn_simt(p, s) == cudaSuccess ? SA_OK : SA_ERR_CUDA;
}

}  // namespace

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
                int32_t* dev_status, void* stream) {
  return attn_fwd_common(q, k, v, o, q_strides, k_strides, v_strides, o_strides, dtype, B, H, Sq, Sk, D, BLOCK_Q,
                         BLOCK_K, mask, mask_strides, packed_bits, bits_stride_b, bits_stride_h, full_ids,
                         full_ids_strides, full_lens, full_lens_strides, part_ids, part_ids_strides, part_lens,
                         part_lens_strides, scale_log2, impl, 1, lse, workspace, workspace_bytes, dev_status, stream);
}

size_t sa_attn_splitkv_workspace_bytes(int dtype, int B, int H, int Sq, int D, int splits) {
  if (!positive(B) || !positive(H) || !positive(Sq) || !positive(D) || !positive(splits)) return 0;
  return split_layout(dtype, B, H, Sq, D, splits).total;
}

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
                        int32_t* dev_status, void* stream) {
  if (splits < 1) return SA_ERR_INVALID_ARGUMENT;
  return attn_fwd_common(q, k, v, o, q_strides, k_strides, v_strides, o_strides, dtype, B, H, Sq, Sk, D, BLOCK_Q,
                         BLOCK_K, mask, mask_strides, packed_bits, bits_stride_b, bits_stride_h, full_ids,
                         full_ids_strides, full_lens, full_lens_strides, part_ids, part_ids_strides, part_lens,
                         part_lens_strides, scale_log2, SA_IMPL_TCGEN05, splits, lse, workspace, workspace_bytes,
                         dev_status, stream);
}

int sa_transpose_lists(const int32_t* full_ids, const int32_t* full_lens,
                       const int32_t* part_ids, const int32_t* part_lens,
                       int planes, int nq, int nk,
                       int32_t* t_full_ids, int32_t* t_full_lens,
                       int32_t* t_part_ids, int32_t* t_part_lens, void* stream) {
  if (full_ids == nullptr || full_lens == nullptr || part_ids == nullptr || part_lens == nullptr ||
      t_full_ids == nullptr || t_full_lens == nullptr || t_part_ids == nullptr || t_part_lens == nullptr)
    return SA_ERR_INVALID_ARGUMENT;
  if (!positive(planes) || !positive(nq) || !positive(nk)) return SA_ERR_INVALID_ARGUMENT;
  if (static_cast<long long>(planes) * nk > 0x7fffffffLL) return SA_ERR_UNSUPPORTED;
  return sa::launch_transpose_lists(full_ids, full_lens, part_ids, part_lens, planes, nq, nk, t_full_ids, t_full_lens,
                                    t_part_ids, t_part_lens, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? SA_OK : SA_ERR_CUDA;
}

size_t sa_attn_bwd_workspace_bytes(int B, int H, int Sq) {
  if (!positive(B) || !positive(H) || !positive(Sq)) return 0;
  return static_cast<size_t>(B) * H * Sq * sizeof(float);
}

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
                int32_t* dev_status, void* stream) {
  sa::AttnBwdParams p;
  std::memset(&p, 0, sizeof(p));
  if (o == nullptr || d_o == nullptr || lse == nullptr || dq == nullptr || dk == nullptr || dv == nullptr ||
      o_strides == nullptr || do_strides == nullptr || dq_strides == nullptr || dk_strides == nullptr ||
      dv_strides == nullptr || mask == nullptr || mask_strides == nullptr)
    return SA_ERR_INVALID_ARGUMENT;
  int rc = fill_attn_params(p.fwd, q, k, v, const_cast<void*>(o), q_strides, k_strides, v_strides, o_strides, dtype,
                            B, H, Sq, Sk, D, BLOCK_Q, BLOCK_K);
  if (rc != SA_OK) return rc;
  if (full_ids == nullptr || full_lens == nullptr || part_ids == nullptr || part_lens == nullptr ||
      full_ids_strides == nullptr || full_lens_strides == nullptr || part_ids_strides == nullptr ||
      part_lens_strides == nullptr || t_full_ids == nullptr || t_full_lens == nullptr || t_part_ids == nullptr ||
      t_part_lens == nullptr || t_full_ids_strides == nullptr || t_full_lens_strides == nullptr ||
      t_part_ids_strides == nullptr || t_part_lens_strides == nullptr)
    return SA_ERR_INVALID_ARGUMENT;
  if (BLOCK_Q % 32 != 0 || BLOCK_K % 32 != 0) return SA_ERR_UNSUPPORTED;
  if (D != 16 && D != 32 && D != 64 && D != 128) return SA_ERR_UNSUPPORTED;
  if (workspace == nullptr || workspace_bytes < sa_attn_bwd_workspace_bytes(B, H, Sq) ||
      reinterpret_cast<uintptr_t>(workspace) % 4 != 0)
    return SA_ERR_WORKSPACE;
  p.fwd.mask = mask; copy_n(p.fwd.ms, mask_strides, 4);
  p.fwd.full_ids = full_ids; copy_n(p.fwd.fis, full_ids_strides, 4);
  p.fwd.full_lens = full_lens; copy_n(p.fwd.fls, full_lens_strides, 3);
  p.fwd.part_ids = part_ids; copy_n(p.fwd.pis, part_ids_strides, 4);
  p.fwd.part_lens = part_lens; copy_n(p.fwd.pls, part_lens_strides, 3);
  p.fwd.scale_log2 = scale_log2;
  p.fwd.lse = const_cast<float*>(lse);
  p.fwd.dev_status = dev_status;
  p.d_o = d_o; copy_n(p.dos, do_strides, 4);
  p.d_lse = d_lse;
  p.dq = dq; p.dk = dk; p.dv = dv;
  copy_n(p.dqs, dq_strides, 4); copy_n(p.dks, dk_strides, 4); copy_n(p.dvs, dv_strides, 4);
  p.dsum = static_cast<float*>(workspace);
  p.t_full_ids = t_full_ids; copy_n(p.tfis, t_full_ids_strides, 4);
  p.t_full_lens = t_full_lens; copy_n(p.tfls, t_full_lens_strides, 3);
  p.t_part_ids = t_part_ids; copy_n(p.tpis, t_part_ids_strides, 4);
  p.t_part_lens = t_part_lens; copy_n(p.tpls, t_part_lens_strides, 3);
  // tensor-core kernels where the inputs allow them (fp16 / bf16, head dim 64 or 128, dense rows), else the CUDA-core ones
  if (sa::attn_bwd_mma_supported(p))
    return sa::launch_attn_bwd_mma(p, static_cast<cudaStream_t>(stream)) == cudaSuccess ? SA_OK : SA_ERR_CUDA;
  return sa::launch_attn_bwd_simt(p, static_cast<cudaStream_t>(stream)) == cudaSuccess ? SA_OK : SA_ERR_CUDA;
}

int sa_selftest_bounded_wait(uint64_t limit_ns, int32_t* dev_status, uint64_t* waited_ns, void* stream) {
  if (dev_status == nullptr) return SA_ERR_INVALID_ARGUMENT;
  if (limit_ns == 0 || limit_ns > 100ull * 1000ull * 1000ull) return SA_ERR_INVALID_ARGUMENT;   // at most 100 ms
  return sa::launch_bounded_wait_probe(limit_ns, dev_status, reinterpret_cast<unsigned long long*>(waited_ns),
                                       static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? SA_OK : SA_ERR_CUDA;
}

}  // extern "C"
