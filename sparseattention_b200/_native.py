"""ctypes binding of ``libsparseattn_b200.so`` (``include/sa_b200.h``) and the two
``torch.library`` custom ops built on it.

There is no CPU implementation and no fallback: the ops accept CUDA tensors only and
raise if the library is missing or a call is outside the supported set.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import List, Optional, Tuple

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SPARSEATTN_B200_LIB") or os.path.join(_PKG_DIR, "libsparseattn_b200.so")

# mirrors of the header's constants
SA_ABI_VERSION = 5
SA_OK = 0
SA_DTYPE_F32, SA_DTYPE_F16, SA_DTYPE_BF16 = 0, 1, 2
SA_IMPL_AUTO, SA_IMPL_SIMT, SA_IMPL_TCGEN05 = 0, 1, 2
SA_DEV_OK, SA_DEV_WAIT_EXPIRED, SA_DEV_BAD_INDEX = 0, 1, 2
SA_WS_UNKNOWN, SA_WS_CLEAN = 0, 1

IMPLS = {"auto": SA_IMPL_AUTO, "simt": SA_IMPL_SIMT, "tcgen05": SA_IMPL_TCGEN05}
_DTYPES = {torch.float32: SA_DTYPE_F32, torch.float16: SA_DTYPE_F16, torch.bfloat16: SA_DTYPE_BF16}

# every symbol the header declares, with its ctypes signature
_i, _i64, _p, _sz, _f = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float
_pi = ctypes.POINTER(ctypes.c_int)
SYMBOLS = {
    "sa_abi_version": (_i, []),
    "sa_status_str": (ctypes.c_char_p, [_i]),
    "sa_unique_planes": (_i, [_i, _i, _i64, _i64, _pi, _pi]),
    "sa_classify_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "sa_classify_mask": (_i, [_p, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _sz, _i, _p]),
    "sa_classify_mask_static": (_i, [_p, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "sa_merge_lists": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "sa_attn_uses_tcgen05": (_i, [_i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _i]),
    "sa_attn_fwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p,
                         _i, _i, _i, _i, _i, _i, _i, _i,
                         _p, _p, _p, _i64, _i64,
                         _p, _p, _p, _p, _p, _p, _p, _p,
                         _f, _i, _p, _p, _sz, _p, _p]),
    "sa_attn_workspace_bytes": (_sz, []),
    "sa_attn_splitkv_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "sa_attn_fwd_splitkv": (_i, [_p, _p, _p, _p, _p, _p, _p, _p,
                                 _i, _i, _i, _i, _i, _i, _i, _i,
                                 _p, _p, _p, _i64, _i64,
                                 _p, _p, _p, _p, _p, _p, _p, _p,
                                 _f, _i, _p, _p, _sz, _p, _p]),
    "sa_selftest_bounded_wait": (_i, [ctypes.c_uint64, _p, _p, _p]),
    "sa_transpose_lists": (_i, [_p, _p, _p, _p, _i, _i, _i, _p, _p, _p, _p, _p]),
    "sa_attn_bwd_workspace_bytes": (_sz, [_i, _i, _i]),
    "sa_attn_bwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p,
                         _p, _p, _p, _p, _p, _p, _p, _p,
                         _i, _i, _i, _i, _i, _i, _i, _i,
                         _p, _p,
                         _p, _p, _p, _p, _p, _p, _p, _p,
                         _p, _p, _p, _p, _p, _p, _p, _p,
                         _f, _p, _sz, _p, _p]),
}

_lib = None


class NativeLibraryError(RuntimeError):
    pass


def load_library():
    """Loads the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NativeLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m sparseattention_b200.build` "
            "(there is no CPU or PyTorch fallback for these ops)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.sa_abi_version() != SA_ABI_VERSION:
        raise NativeLibraryError("libsparseattn_b200.so has a different ABI version; rebuild it")
    _lib = lib
    return lib


def status_str(rc: int) -> str:
    return load_library().sa_status_str(rc).decode()


def _check(rc: int, what: str) -> None:
    if rc != SA_OK:
        msg = f"{what}: {status_str(rc)} (status {rc})"
        if rc == -2:
            raise NotImplementedError(msg)
        if rc in (-1, -3):
            raise ValueError(msg)
        raise RuntimeError(msg)


def _strides(t: torch.Tensor):
    arr = (ctypes.c_int64 * t.dim())(*t.stride())
    return arr


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("sparseattention_b200 ops run on CUDA tensors only (no CPU fallback)")


# ------------------------------------------------------------------------------- stage 1

def unique_planes(mask: torch.Tensor) -> Tuple[int, int]:
    B, H = mask.shape[0], mask.shape[1]
    bu = 1 if (mask.stride(0) == 0 or B == 1) else B
    hu = 1 if (mask.stride(1) == 0 or H == 1) else H
    return bu, hu


def _canonical_mask(mask: torch.Tensor) -> torch.Tensor:
    """A view (or, if the layout cannot be streamed with 16-byte loads, a copy) of the
    mask whose size-1 / broadcast leading dims carry stride 0."""
    B, H, Sq, Sk = mask.shape
    bu, hu = unique_planes(mask)
    base = mask[: bu, : hu]
    ok = (base.stride(3) == 1 and base.stride(2) % 16 == 0 and base.stride(2) >= Sk
          and base.data_ptr() % 16 == 0
          and (bu == 1 or base.stride(0) % 16 == 0) and (hu == 1 or base.stride(1) % 16 == 0))
    if not ok:
        base = base.contiguous()
    return base


# Classifier workspaces kept between calls, one per (device, stream): the kernel needs its workspace
# zero-filled and leaves it zero-filled, so a kept workspace is cleared once, when it is made.
_CLASSIFY_WS = {}


def _classify_workspace(dev: torch.device, n_bytes: int) -> torch.Tensor:
    """A zero-filled workspace of at least ``n_bytes`` for the current stream of ``dev``.  While a CUDA
    graph is being captured a fresh one is made inside the capture instead (memory that a graph's pool
    owns must not be kept for use outside it)."""
    if torch.cuda.is_current_stream_capturing():
        return torch.zeros((n_bytes,), dtype=torch.uint8, device=dev)
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _CLASSIFY_WS.get(key)
    if ws is None or ws.numel() < n_bytes:
        ws = torch.zeros((max(n_bytes, 1 << 16),), dtype=torch.uint8, device=dev)
        _CLASSIFY_WS[key] = ws
    return ws


def _plain(*tensors: torch.Tensor) -> bool:
    """True when the kernels may be called without going through the dispatcher: eager mode, ordinary
    tensors.  (The dispatcher of a Python custom op costs tens of microseconds of host time per call, more
    than the kernels of a small problem take; tracing, fake tensors and autograd do need it.)"""
    return not torch.compiler.is_compiling() and all(type(t) is torch.Tensor for t in tensors)


def _classify_mask_impl(mask: torch.Tensor, block_q: int, block_k: int,
                        with_bits: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """mask: bool [Bu,Hu,Sq,Sk] holding only the distinct planes.  Returns
    (full_ids, full_lens, part_ids, part_lens, packed_bits) for those planes."""
    _require_cuda(mask)
    if mask.dtype != torch.bool:
        raise TypeError("mask must be a bool tensor")             # mask_utils.py:18
    lib = load_library()
    Bu, Hu, Sq, Sk = mask.shape
    if Sq % block_q != 0 or Sk % block_k != 0:
        raise ValueError("Sq and Sk must be multiples of BLOCK_Q and BLOCK_K")   # mask_utils.py:89-90
    nq, nk = Sq // block_q, Sk // block_k
    dev = mask.device
    with torch.cuda.device(dev):
        full_ids = torch.empty((Bu, Hu, nq, nk), dtype=torch.int32, device=dev)
        part_ids = torch.empty((Bu, Hu, nq, nk), dtype=torch.int32, device=dev)
        full_lens = torch.empty((Bu, Hu, nq), dtype=torch.int32, device=dev)
        part_lens = torch.empty((Bu, Hu, nq), dtype=torch.int32, device=dev)
        bits = (torch.empty((Bu, Hu, Sk // 32, Sq), dtype=torch.int32, device=dev) if with_bits
                else torch.empty((0,), dtype=torch.int32, device=dev))
        ws_bytes = lib.sa_classify_workspace_bytes(Bu, Hu, Sq, Sk)
        ws = _classify_workspace(dev, ws_bytes)
        sb = mask.stride(0) if Bu > 1 else 0
        sh = mask.stride(1) if Hu > 1 else 0
        rc = lib.sa_classify_mask(mask.data_ptr(), sb, sh, mask.stride(2), mask.stride(3),
                                  Bu, Hu, Sq, Sk, block_q, block_k,
                                  full_ids.data_ptr(), full_lens.data_ptr(), part_ids.data_ptr(), part_lens.data_ptr(),
                                  bits.data_ptr() if with_bits else None,
                                  ws.data_ptr(), ws.numel(), SA_WS_CLEAN, _stream_ptr(dev))
    _check(rc, "sa_classify_mask")
    return full_ids, full_lens, part_ids, part_lens, bits


classify_mask_op = torch.library.custom_op("sparseattention::classify_mask", mutates_args=())(_classify_mask_impl)


@classify_mask_op.register_fake
def _(mask, block_q, block_k, with_bits):
    Bu, Hu, Sq, Sk = mask.shape
    nq, nk = Sq // block_q, Sk // block_k
    ids = lambda: mask.new_empty((Bu, Hu, nq, nk), dtype=torch.int32)
    lens = lambda: mask.new_empty((Bu, Hu, nq), dtype=torch.int32)
    bits = mask.new_empty((Bu, Hu, Sk // 32, Sq) if with_bits else (0,), dtype=torch.int32)
    return ids(), lens(), ids(), lens(), bits


def classify(mask: torch.Tensor, block_q: int, block_k: int, with_bits: bool = True):
    """Classifies a [B,H,Sq,Sk] bool mask (broadcast dims allowed).  Returns the five
    tensors of :func:`classify_mask_op` computed over the distinct planes only."""
    if mask.dim() != 4:
        raise ValueError("mask must be [B,H,Sq,Sk]")
    mask = _canonical_mask(mask)
    fn = _classify_mask_impl if _plain(mask) else classify_mask_op
    return fn(mask, int(block_q), int(block_k), bool(with_bits))


def merge_lists(full_ids: torch.Tensor, full_lens: torch.Tensor, part_ids: torch.Tensor, part_lens: torch.Tensor,
                block_q_in: int, block_k: int, ratio: int, bits: torch.Tensor):
    """Lists for query blocks of ``block_q_in`` rows ([P0,P1,nq_in,nk] / [P0,P1,nq_in], contiguous int32,
    distinct planes only) -> lists for blocks ``ratio`` times taller.  ``bits`` ([P0,P1,Sk/32,Sq]) is
    patched in place so that it says what the short lists say (see ``sa_merge_lists``)."""
    _require_cuda(full_ids, full_lens, part_ids, part_lens, bits)
    lib = load_library()
    P0, P1, nq_in, nk = full_ids.shape
    dev = full_ids.device
    with torch.cuda.device(dev):
        out_ids = lambda: torch.empty((P0, P1, nq_in // ratio, nk), dtype=torch.int32, device=dev)
        out_lens = lambda: torch.empty((P0, P1, nq_in // ratio), dtype=torch.int32, device=dev)
        f_ids, p_ids, f_lens, p_lens = out_ids(), out_ids(), out_lens(), out_lens()
        rc = lib.sa_merge_lists(full_ids.data_ptr(), full_lens.data_ptr(), part_ids.data_ptr(), part_lens.data_ptr(),
                                P0 * P1, nq_in, nk, ratio, block_q_in, block_k,
                                f_ids.data_ptr(), f_lens.data_ptr(), p_ids.data_ptr(), p_lens.data_ptr(),
                                bits.data_ptr(), _stream_ptr(dev))
    _check(rc, "sa_merge_lists")
    return f_ids, f_lens, p_ids, p_lens


# ------------------------------------------------------------------------------- stage 2

def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """Q/K/V as the kernels want them: unit stride in D; otherwise a contiguous copy."""
    if t.stride(-1) != 1:
        return t.contiguous()
    return t


def _attn_fwd_impl(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, bits: torch.Tensor,
                full_ids: torch.Tensor, full_lens: torch.Tensor, part_ids: torch.Tensor, part_lens: torch.Tensor,
                block_q: int, block_k: int, impl: int, check_status: bool,
                with_lse: bool, splits: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block-sparse attention forward over precomputed lists.  ``mask`` [B,H,Sq,Sk] and the
    list tensors ([B,H,nq,nk] / [B,H,nq]) may be expanded views; ``bits`` is the packed plane
    [Bu,Hu,Sk/32,Sq] (or an empty tensor when absent).  Returns (O, LSE): LSE is float32 [B,H,Sq],
    the natural-log sum of exp of a row's scaled scores over its attended keys (-inf for none), or
    an empty tensor when ``with_lse`` is False.  ``splits`` > 1 cuts every walk over the lists into that
    many ranges that run side by side and are combined by a second kernel (tensor-core kernel only)."""
    _require_cuda(q, k, v, mask, full_ids, full_lens, part_ids, part_lens)
    lib = load_library()
    B, H, Sq, D = q.shape
    Sk = k.shape[-2]
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share one of float32 / float16 / bfloat16")
    if tuple(k.shape) != (B, H, Sk, D) or tuple(v.shape) != (B, H, Sk, D):
        raise ValueError("k and v must be [B,H,Sk,D] with the batch and head counts of q")
    if tuple(mask.shape) != (B, H, Sq, Sk):
        raise ValueError("mask must be (expandable to) [B,H,Sq,Sk]")
    if Sq % block_q != 0 or Sk % block_k != 0:
        raise ValueError("Sq and Sk must be multiples of BLOCK_Q and BLOCK_K")
    scale_log2 = D ** -0.5 / math.log(2)                        # sparse_attn_kernel.py:152
    dev = q.device
    with torch.cuda.device(dev):
        o = torch.empty((B, H, Sq, D), dtype=q.dtype, device=dev)    # sparse_attn_kernel.py:165
        has_bits = bits.numel() > 0
        if has_bits:
            bsb = bits.stride(0) if bits.shape[0] > 1 else 0
            bsh = bits.stride(1) if bits.shape[1] > 1 else 0
        else:
            bsb = bsh = 0
        status = torch.zeros((1,), dtype=torch.int32, device=dev) if check_status else None
        lse = torch.empty((B, H, Sq) if with_lse else (0,), dtype=torch.float32, device=dev)
        if splits > 1:
            ws_bytes = int(lib.sa_attn_splitkv_workspace_bytes(_DTYPES[q.dtype], B, H, Sq, D, splits))
        else:
            ws_bytes = int(lib.sa_attn_workspace_bytes())
        ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)        # the counter in it is cleared by the call
        head = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                _strides(q), _strides(k), _strides(v), _strides(o),
                _DTYPES[q.dtype], B, H, Sq, Sk, D, block_q, block_k,
                mask.data_ptr(), _strides(mask),
                bits.data_ptr() if has_bits else None, bsb, bsh,
                full_ids.data_ptr(), _strides(full_ids), full_lens.data_ptr(), _strides(full_lens),
                part_ids.data_ptr(), _strides(part_ids), part_lens.data_ptr(), _strides(part_lens),
                scale_log2)
        tail = (lse.data_ptr() if with_lse else None, ws.data_ptr(), ws_bytes,
                status.data_ptr() if check_status else None, _stream_ptr(dev))
        if splits > 1:
            rc = lib.sa_attn_fwd_splitkv(*head, splits, *tail)
        else:
            rc = lib.sa_attn_fwd(*head, impl, *tail)
    _check(rc, "sa_attn_fwd_splitkv" if splits > 1 else "sa_attn_fwd")
    if check_status:
        code = int(status.item())
        if code != SA_DEV_OK:
            raise RuntimeError({SA_DEV_WAIT_EXPIRED: "attention kernel: a bounded device-side wait expired",
                                SA_DEV_BAD_INDEX: "attention kernel: kv-block id out of range in a list"}.get(
                                    code, f"attention kernel: device status {code}"))
    return o, lse


attn_fwd_op = torch.library.custom_op("sparseattention::attn_fwd", mutates_args=())(_attn_fwd_impl)


def attn_fwd(*args, differentiable: bool):
    """The attention forward: through the registered op when a backward pass may follow (or under tracing),
    directly otherwise."""
    if not differentiable and _plain(*args[:9]):
        return _attn_fwd_impl(*args)
    return attn_fwd_op(*args)


@attn_fwd_op.register_fake
def _(q, k, v, mask, bits, full_ids, full_lens, part_ids, part_lens, block_q, block_k, impl, check_status,
      with_lse, splits=1):
    B, H, Sq, _ = q.shape
    return q.new_empty(q.shape), q.new_empty((B, H, Sq) if with_lse else (0,), dtype=torch.float32)


# ------------------------------------------------------------------------------- backward of stage 2

def transpose_lists(full_ids: torch.Tensor, full_lens: torch.Tensor, part_ids: torch.Tensor, part_lens: torch.Tensor):
    """kv-major lists from query-major ones: ``[P0,P1,nq,nk]`` ids / ``[P0,P1,nq]`` lengths (contiguous int32,
    distinct planes) -> ``[P0,P1,nk,nq]`` ids (ascending query blocks, tails -1) and ``[P0,P1,nk]`` lengths,
    for the full and for the partial lists."""
    _require_cuda(full_ids, full_lens, part_ids, part_lens)
    lib = load_library()
    P0, P1, nq, nk = full_ids.shape
    dev = full_ids.device
    with torch.cuda.device(dev):
        ids = lambda: torch.empty((P0, P1, nk, nq), dtype=torch.int32, device=dev)
        lens = lambda: torch.empty((P0, P1, nk), dtype=torch.int32, device=dev)
        tf_ids, tp_ids, tf_lens, tp_lens = ids(), ids(), lens(), lens()
        rc = lib.sa_transpose_lists(full_ids.data_ptr(), full_lens.data_ptr(), part_ids.data_ptr(), part_lens.data_ptr(),
                                    P0 * P1, nq, nk, tf_ids.data_ptr(), tf_lens.data_ptr(), tp_ids.data_ptr(),
                                    tp_lens.data_ptr(), _stream_ptr(dev))
    _check(rc, "sa_transpose_lists")
    return tf_ids, tf_lens, tp_ids, tp_lens


@torch.library.custom_op("sparseattention::attn_bwd", mutates_args=())
def attn_bwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, d_o: torch.Tensor,
                lse: torch.Tensor, d_lse: Optional[torch.Tensor], mask: torch.Tensor,
                full_ids: torch.Tensor, full_lens: torch.Tensor, part_ids: torch.Tensor, part_lens: torch.Tensor,
                t_full_ids: torch.Tensor, t_full_lens: torch.Tensor, t_part_ids: torch.Tensor, t_part_lens: torch.Tensor,
                block_q: int, block_k: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of :func:`attn_fwd_op` with respect to q, k, v (``sa_attn_bwd``): ``o`` and ``lse`` are the
    forward's outputs, ``d_o`` / ``d_lse`` their incoming gradients, the lists the ones the forward walked and
    their kv-major transposes (all may be expanded views)."""
    _require_cuda(q, k, v, o, d_o, lse, mask)
    lib = load_library()
    B, H, Sq, D = q.shape
    Sk = k.shape[-2]
    dev = q.device
    scale_log2 = D ** -0.5 / math.log(2)
    with torch.cuda.device(dev):
        lse = lse.contiguous()
        gl = None if d_lse is None else d_lse.to(torch.float32).contiguous()
        dq = torch.empty((B, H, Sq, D), dtype=q.dtype, device=dev)
        dk = torch.empty((B, H, Sk, D), dtype=q.dtype, device=dev)
        dv = torch.empty((B, H, Sk, D), dtype=q.dtype, device=dev)
        ws_bytes = int(lib.sa_attn_bwd_workspace_bytes(B, H, Sq))
        ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)
        rc = lib.sa_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(),
                             lse.data_ptr(), None if gl is None else gl.data_ptr(),
                             dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                             _strides(q), _strides(k), _strides(v), _strides(o), _strides(d_o),
                             _strides(dq), _strides(dk), _strides(dv),
                             _DTYPES[q.dtype], B, H, Sq, Sk, D, block_q, block_k,
                             mask.data_ptr(), _strides(mask),
                             full_ids.data_ptr(), _strides(full_ids), full_lens.data_ptr(), _strides(full_lens),
                             part_ids.data_ptr(), _strides(part_ids), part_lens.data_ptr(), _strides(part_lens),
                             t_full_ids.data_ptr(), _strides(t_full_ids), t_full_lens.data_ptr(), _strides(t_full_lens),
                             t_part_ids.data_ptr(), _strides(t_part_ids), t_part_lens.data_ptr(), _strides(t_part_lens),
                             scale_log2, ws.data_ptr(), ws_bytes, None, _stream_ptr(dev))
    _check(rc, "sa_attn_bwd")
    return dq, dk, dv


@attn_bwd_op.register_fake
def _(q, k, v, o, d_o, lse, d_lse, mask, full_ids, full_lens, part_ids, part_lens, t_full_ids, t_full_lens,
      t_part_ids, t_part_lens, block_q, block_k):
    return q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape)


def _distinct_planes(t: torch.Tensor) -> torch.Tensor:
    bu = 1 if (t.shape[0] == 1 or t.stride(0) == 0) else t.shape[0]
    hu = 1 if (t.shape[1] == 1 or t.stride(1) == 0) else t.shape[1]
    return t[:bu, :hu]


def _attn_setup_context(ctx, inputs, output):
    q, k, v, mask, bits, full_ids, full_lens, part_ids, part_lens, block_q, block_k, impl, check_status, with_lse = \
        inputs[:14]
    o, lse = output
    if not with_lse:
        raise RuntimeError("the attention op was called without its log-sum-exp output: no backward is possible "
                           "(sparse_attention asks for it whenever an input requires grad)")
    ctx.save_for_backward(q, k, v, o, lse, mask, full_ids, full_lens, part_ids, part_lens)
    ctx.blocks = (block_q, block_k)


def _attn_backward(ctx, grad_o, grad_lse):
    q, k, v, o, lse, mask, full_ids, full_lens, part_ids, part_lens = ctx.saved_tensors
    block_q, block_k = ctx.blocks
    B, H = q.shape[0], q.shape[1]
    # kv-major lists, built over the distinct planes of the (possibly expanded) lists
    planes = [_distinct_planes(t).contiguous() for t in (full_ids, full_lens, part_ids, part_lens)]
    if len({tuple(t.shape[:2]) for t in planes}) != 1:
        planes = [t.expand(B, H, *t.shape[2:]).contiguous() for t in (full_ids, full_lens, part_ids, part_lens)]
    t_lists = transpose_lists(*planes)
    ex = lambda t: t.expand(*((B, H) + tuple(t.shape[2:])))
    dq, dk, dv = attn_bwd_op(q, k, v, o, grad_o.contiguous(), lse, grad_lse, mask, full_ids, full_lens, part_ids,
                             part_lens, ex(t_lists[0]), ex(t_lists[1]), ex(t_lists[2]), ex(t_lists[3]),
                             block_q, block_k)
    return dq, dk, dv, None, None, None, None, None, None, None, None, None, None, None, None


attn_fwd_op.register_autograd(_attn_backward, setup_context=_attn_setup_context)


def uses_tcgen05(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_q: int, block_k: int,
                 has_bits: bool = True) -> bool:
    """Whether ``impl='auto'`` runs the tcgen05 kernel for these tensors."""
    lib = load_library()
    if q.dtype not in _DTYPES:
        return False
    return bool(lib.sa_attn_uses_tcgen05(_DTYPES[q.dtype], q.shape[-1], block_q, block_k, q.shape[-2], k.shape[-2],
                                         q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                         _strides(q), _strides(k), _strides(v), int(has_bits)))
