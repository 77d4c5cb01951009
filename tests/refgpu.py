"""ctypes access to oracle/_ref/libref_gpu.so: the reference's own CUDA kernels
compiled for sm_100a from their own sources.  Test helper only."""
import ctypes as C
from pathlib import Path

_PATH = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_gpu.so"
_lib = None


def load():
    global _lib
    if _lib is None:
        if not _PATH.exists():
            return None
        _lib = C.CDLL(str(_PATH))
    return _lib
