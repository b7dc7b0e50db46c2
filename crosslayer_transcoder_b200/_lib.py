"""ctypes binding of ``libclt_b200.so``.

The argument types of every entry point are read from ``include/clt_b200.h`` so the
binding cannot drift from the declared C ABI.  There is no fallback: when the
library is missing, cannot be loaded, or the current device is not sm_100, the
first use raises.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path
from typing import Dict, List, Tuple

import torch

PKG = Path(__file__).resolve().parent
HEADER = PKG.parent / "include" / "clt_b200.h"
LIB_PATH = PKG / "libclt_b200.so"

_CTYPES = {
    "int": ctypes.c_int,
    "float": ctypes.c_float,
    "int64_t": ctypes.c_int64,
    "clt_stream_t": ctypes.c_void_p,
}


def parse_header(path: Path = HEADER) -> Dict[str, Tuple[object, List[Tuple[str, object]]]]:
    """{name: (restype, [(argname, ctype), ...])} for every ``clt_*`` prototype."""
    text = re.sub(r"/\*.*?\*/", "", path.read_text(), flags=re.S)
    protos = {}
    for m in re.finditer(r"(const\s+char\s*\*|int)\s+(clt_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1), m.group(2), m.group(3).strip()
        restype = ctypes.c_char_p if "char" in ret else ctypes.c_int
        arglist = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                if "*" in a:
                    arglist.append((a.split("*")[-1].strip(), ctypes.c_void_p))
                else:
                    typ, an = a.rsplit(" ", 1)
                    arglist.append((an, _CTYPES[typ.replace("const ", "").strip()]))
        protos[name] = (restype, arglist)
    return protos


class CltError(RuntimeError):
    pass


class _Lib:
    def __init__(self):
        if not LIB_PATH.exists():
            raise CltError(
                f"{LIB_PATH} is missing: build it with `python -m crosslayer_transcoder_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        self.cdll = ctypes.CDLL(str(LIB_PATH))
        self.protos = parse_header()
        for name, (restype, args) in self.protos.items():
            fn = getattr(self.cdll, name)          # AttributeError if a declared symbol is not exported
            fn.restype = restype
            fn.argtypes = [t for _, t in args]
        self._device_ok = set()

    def last_error(self) -> str:
        s = self.cdll.clt_last_error()
        return s.decode() if s else ""

    def check_device(self):
        if not torch.cuda.is_available():
            raise CltError("no CUDA device: this package runs on B200 (sm_100a) only and has no CPU fallback")
        dev = torch.cuda.current_device()
        if dev not in self._device_ok:
            if self.cdll.clt_device_check() != 0:
                raise CltError(self.last_error())
            self._device_ok.add(dev)

    def call(self, name: str, *args):
        """Call an ``int``-returning entry point; tensors are passed as their data pointers."""
        conv = []
        for a in args:
            if isinstance(a, torch.Tensor):
                conv.append(a.data_ptr())
            else:
                conv.append(a)
        rc = getattr(self.cdll, name)(*conv)
        if rc != 0:
            raise CltError(f"{name} failed ({rc}): {self.last_error()}")


_lib = None


def lib() -> _Lib:
    global _lib
    if _lib is None:
        _lib = _Lib()
    return _lib


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

STATUS_NAMES = {
    0x10: "the MMA warp gave up waiting for a TMA stage",
    0x11: "the TMA warp gave up waiting for a free stage",
    0x12: "the epilogue gave up waiting for an accumulator",
    0x13: "the MMA warp gave up waiting for the epilogue",
    0x20: "an index read from memory was out of range",
    0x21: "a fixed-capacity list overflowed",
}


def check_status(status: torch.Tensor, where: str = ""):
    """Read the device status word (synchronises) and raise if a kernel reported a failure."""
    code = int(status.item())
    if code != 0:
        status.zero_()
        raise CltError(f"device status {code:#x} {where}: {STATUS_NAMES.get(code, 'unknown code')}")
