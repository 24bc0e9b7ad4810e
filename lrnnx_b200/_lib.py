"""ctypes binding of liblrnnx_b200.so.

The argument-block layouts are parsed from ``include/lrnnx_b200.h`` so the
header stays the single description of the ABI; ``check_layout`` compares every
parsed size against ``b200_sizeof`` of the loaded library.

There is no fallback: if the shared library is missing, ``lib()`` raises
``RuntimeError`` telling the user to build it.
"""
from __future__ import annotations

import ctypes
import re
from functools import lru_cache
from pathlib import Path

_PKG = Path(__file__).resolve().parent
HEADER = _PKG.parent / "include" / "lrnnx_b200.h"
LIB_PATH = _PKG / "lib" / "liblrnnx_b200.so"

ENTRY_POINTS = (
    "b200_last_error", "b200_abi_version", "b200_sizeof", "b200_device_status", "b200_s4_bwd_scratch_bytes",
    "b200_selscan_stage_states",
    "b200_selscan_fwd", "b200_selscan_bwd", "b200_selscan_fixup", "b200_selscan_fold",
    "b200_selscan_adjoint_summary",
    "b200_simpscan_fwd", "b200_simpscan_bwd",
    "b200_ssu_step", "b200_s5_step",
    "b200_cauchy_fwd", "b200_cauchy_bwd", "b200_cauchy_bwd_static", "b200_vand_fwd", "b200_vand_bwd",
    "b200_conv1d_fwd", "b200_conv1d_bwd", "b200_conv1d_update", "b200_rmsnorm_fwd", "b200_rmsnorm_bwd",
    "b200_cgemm_wx", "b200_cgemm_planes", "b200_cgemm_grad",
    "b200_xent_fwd", "b200_xent_bwd", "b200_skinny_linear",
)

_SCALARS = {"int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64, "uint32_t": ctypes.c_uint32,
            "float": ctypes.c_float}


def _strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


@lru_cache(maxsize=None)
def parse_header() -> tuple[dict, dict, list]:
    """Return (structs, enums, functions) declared in the public header."""
    text = _strip_comments(HEADER.read_text())
    enums: dict[str, int] = {}
    for body in re.findall(r"enum\s*\{(.*?)\}", text, flags=re.S):
        nxt = 0
        for item in body.split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, val = (s.strip() for s in item.split("="))
                nxt = int(val, 0)
            else:
                name = item
            enums[name] = nxt
            nxt += 1
    structs: dict[str, type] = {}
    for name, body in re.findall(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*\w+\s*;", text, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = " ".join(decl.split())
            if not decl:
                continue
            decl = decl.replace("const ", "")
            base, rest = decl.split(" ", 1)
            for var in rest.split(","):
                var = var.strip()
                is_ptr = var.startswith("*")
                var = var.lstrip("* ")
                if is_ptr:
                    ctype = ctypes.c_void_p
                elif base in _SCALARS:
                    ctype = _SCALARS[base]
                elif base in structs:
                    ctype = structs[base]
                else:
                    raise ValueError(f"cannot parse field '{decl}' of {name}")
                fields.append((var, ctype))
        structs[name] = type(name, (ctypes.Structure,), {"_fields_": fields})
    functions = re.findall(r"^\s*(?:const\s+char\s*\*|int|int64_t)\s*(b200_\w+)\s*\(", text, flags=re.M)
    return structs, enums, functions


def struct(name: str) -> type:
    return parse_header()[0][name]


def enum(name: str) -> int:
    return parse_header()[1][name]


_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built. "
            "Run `python -m lrnnx_b200.build` (needs nvcc); there is no CPU or PyTorch fallback."
        )
    handle = ctypes.CDLL(str(LIB_PATH))
    handle.b200_last_error.restype = ctypes.c_char_p
    handle.b200_last_error.argtypes = []
    handle.b200_abi_version.restype = ctypes.c_int
    handle.b200_sizeof.restype = ctypes.c_int
    handle.b200_sizeof.argtypes = [ctypes.c_char_p]
    handle.b200_device_status.restype = ctypes.c_int
    handle.b200_device_status.argtypes = []
    handle.b200_s4_bwd_scratch_bytes.restype = ctypes.c_int64
    handle.b200_s4_bwd_scratch_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    handle.b200_selscan_stage_states.restype = ctypes.c_int
    handle.b200_selscan_stage_states.argtypes = [ctypes.c_void_p]
    for fn in ENTRY_POINTS[6:]:
        f = getattr(handle, fn)
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    _lib = handle
    check_layout()
    return _lib


def check_layout() -> None:
    structs = parse_header()[0]
    for name, st in structs.items():
        want = _lib.b200_sizeof(name.encode())
        if want != ctypes.sizeof(st):
            raise RuntimeError(f"ABI mismatch for {name}: header says {ctypes.sizeof(st)} bytes, library {want}")


def call(fn_name: str, args: ctypes.Structure, stream: int) -> None:
    """Invoke an entry point; raise RuntimeError carrying the library's message on failure."""
    rc = getattr(lib(), fn_name)(ctypes.byref(args), ctypes.c_void_p(stream))
    if rc != 0:
        msg = lib().b200_last_error().decode(errors="replace")
        raise RuntimeError(f"{fn_name} failed (status {rc}): {msg}")
