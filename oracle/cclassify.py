"""ctypes front end of ``classify_ref.c`` (test infrastructure; see that file)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

from .classifier import OracleMetadata

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_classify.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "classify_ref.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle_classify.so"], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_LIB_PATH)
        i64, p = ctypes.c_int64, ctypes.c_void_p
        lib.sa_oracle_classify.argtypes = [p, i64, i64, i64, i64, i64, p, p, p, p]
        lib.sa_oracle_classify.restype = ctypes.c_int
        lib.sa_oracle_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def threads() -> int:
    return int(_load().sa_oracle_threads())


def classify(mask: np.ndarray, block_q: int, block_k: int) -> OracleMetadata:
    """mask: bool/uint8 [B,H,Sq,Sk] -> lists, via the C restatement."""
    lib = _load()
    B, H, Sq, Sk = mask.shape
    m = np.ascontiguousarray(mask).view(np.uint8)
    nq, nk = Sq // block_q, Sk // block_k
    f_ids = np.empty((B, H, nq, nk), np.int32)
    p_ids = np.empty((B, H, nq, nk), np.int32)
    f_lens = np.empty((B, H, nq), np.int32)
    p_lens = np.empty((B, H, nq), np.int32)
    rc = lib.sa_oracle_classify(m.ctypes.data, B * H, Sq, Sk, block_q, block_k,
                                f_ids.ctypes.data, f_lens.ctypes.data,
                                p_ids.ctypes.data, p_lens.ctypes.data)
    if rc != 0:
        raise ValueError("Sq/Sk must be multiples of the block sizes")
    return OracleMetadata(f_ids, f_lens, p_ids, p_lens)
