"""Loader (and builder) of the native library behind the C ABI of ``include/lcgemm_b200.h``.

The device code of this package lives in one shared library built from
``csrc/*.cu`` for sm_100a.  There is no other implementation of the hot path:
if the library cannot be loaded every operator of the package raises.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

_PKG = Path(__file__).resolve().parent
CSRC = _PKG.parent / "csrc"
INCLUDE = _PKG.parent.parent / "include"
LIB_DIR = _PKG / "_lib"
# LCGEMM_B200_LIB points the loader at another build of the same sources (an A/B comparison).
LIB_PATH = Path(os.environ.get("LCGEMM_B200_LIB") or LIB_DIR / "liblcgemm_b200.so")
SOURCES = ("lcg_scheme.cu", "lcg_simt.cu", "lcg_gemm.cu", "lcg_static.cu", "lcg_peer.cu")

OK = 0
ERR_BAD_ARG, ERR_UNSUPPORTED_SHAPE, ERR_MISALIGNED, ERR_SCHEME, ERR_CUDA, ERR_DEVICE_TIMEOUT = (
    -1, -2, -3, -4, -5, -6)
SCHEDULE_ALL_RANKS, SCHEDULE_RANK_SPLIT, SCHEDULE_HYBRID = 0, 1, 2

_c = ctypes
_vp, _i64, _i32, _f32 = _c.c_void_p, _c.c_int64, _c.c_int, _c.c_float

# name -> (restype, argtypes); every symbol the header declares.
SIGNATURES = {
    "lcg_version": (_i32, []),
    "lcg_last_error": (_c.c_char_p, []),
    "lcg_scheme_create": (_i32, [_vp, _vp, _vp, _i32, _vp, _c.POINTER(_vp)]),
    "lcg_scheme_destroy": (None, [_vp]),
    "lcg_scheme_plan": (_i32, [_vp, _vp, _vp]),
    "lcg_plane_geometry": (_i32, [_i64, _i64, _i32, _c.POINTER(_i64), _c.POINTER(_i64),
                                  _c.POINTER(_i64)]),
    "lcg_prepare_b": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "lcg_a_planes": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "lcg_norm_planes": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _vp, _vp, _i64, _vp]),
    "lcg_swiglu_planes": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "lcg_gemm_dense": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _vp, _vp]),
    "lcg_gemm_r7": (_i32, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _i32,
                           _vp, _vp]),
    "lcg_gemm_r7_fused": (_i32, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _i32,
                                 _vp, _vp]),
    "lcg_gemm_r7_fused_supported": (_i32, [_vp, _i64, _i64, _i64]),
    "lcg_gemm_r7_ahead": (_i32, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _i32, _i32,
                                 _vp, _vp]),
    "lcg_gemm_r7_ahead_scratch_bytes": (_i64, [_vp, _i64, _i64]),
    "lcg_gemm_r7_slab": (_i32, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _i32,
                                _i32, _i32, _i32, _vp, _vp]),
    "lcg_gate_up_chain": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64,
                                 _vp, _i64, _vp, _i64, _i32, _i32, _vp, _vp]),
    "lcg_gate_up_chain_init": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64,
                                      _vp, _i64, _vp, _i64, _vp, _i32, _i32, _vp, _vp]),
    "lcg_gemm_r7_push": (_i32, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp, _i32, _i32,
                                _i64, _i32, _vp, _vp]),
    "lcg_peer_barrier": (_i32, [_vp, _i32, _i32, _c.c_uint32, _i64, _vp, _vp]),
    "lcg_reduce_gather": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "lcg_selftest_wait_timeout": (_i32, [_vp, _i64, _vp, _vp]),
    "lcg_gemm_r7_static": (_i32, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _i32,
                                  _vp, _vp]),
    "lcg_static_scratch_bytes": (_i64, []),
    "lcg_static_reserve": (_i32, []),
    "lcg_add_rmsnorm": (_i32, [_vp, _vp, _vp, _i64, _i64, _f32, _vp, _vp, _vp]),
    "lcg_swiglu": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "lcg_add": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "lcg_launch_count": (_i64, []),
    "lcg_describe_gemm": (_i32, [_i64, _i64, _i64, _i32, _i32, _i32, _c.c_char_p, _i32]),
}

_lib = None


def nvcc_command(out: Path = LIB_PATH, extra: tuple = ()) -> list:
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    return ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
            "-std=c++17", "-shared", "-Xcompiler", "-fPIC", f"-I{INCLUDE}", *extra,
            "-o", str(out), *srcs]


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``csrc/*.cu`` into ``_lib/liblcgemm_b200.so`` (cross-compiles without a GPU)."""
    LIB_DIR.mkdir(exist_ok=True)
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    deps = srcs + sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    if not force and LIB_PATH.exists():
        newest = max(p.stat().st_mtime for p in deps)
        if LIB_PATH.stat().st_mtime >= newest:
            return LIB_PATH
    cmd = nvcc_command(extra=("-Xptxas", "-v") if verbose else ())
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        print(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return LIB_PATH


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            if os.environ.get("LCGEMM_B200_AUTOBUILD", "0") == "1":
                build()
            else:
                raise RuntimeError(
                    f"{LIB_PATH} is missing: the CUDA library of lcgemm_b200 has not been built "
                    f"(run `python -c 'import __graft_entry__ as g; g.build()'` at the repository "
                    f"root). There is no fallback implementation of this path.")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue            # optional entry points are checked by their callers
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


_ERRORS = {
    ERR_BAD_ARG: ValueError,
    ERR_UNSUPPORTED_SHAPE: ValueError,
    ERR_MISALIGNED: ValueError,
    ERR_SCHEME: ValueError,
    ERR_CUDA: RuntimeError,
    ERR_DEVICE_TIMEOUT: RuntimeError,
}


def check(code: int) -> None:
    """Turn a negative status into the exception type the reference raises for that failure
    (``ValueError`` for shapes and arguments, ``RuntimeError`` for state and CUDA)."""
    if code != OK:
        msg = lib().lcg_last_error().decode("utf-8", "replace")
        raise _ERRORS.get(code, RuntimeError)(f"lcgemm_b200 error {code}: {msg}")


class NativeScheme:
    """Owns an ``lcg_scheme_t*`` built from a host-side :class:`lcgemm.scheme.Scheme`."""

    _cache: dict = {}

    def __init__(self, scheme):
        if tuple(scheme.shape) != (2, 2, 2):
            raise ValueError(f"the B200 kernels implement 2x2x2 schemes, got {scheme.shape}")
        flat = lambda rows: (ctypes.c_int8 * (len(rows) * 4))(*[v for row in rows for v in row])
        a, b, c = flat(scheme.a), flat(scheme.b), flat(scheme.c)
        clear = (ctypes.c_int8 * scheme.rank)(*scheme.clear) if scheme.has_postsum else None
        handle = ctypes.c_void_p()
        check(lib().lcg_scheme_create(a, b, c, scheme.rank, clear, ctypes.byref(handle)))
        self.handle = handle
        self.scheme = scheme

    @classmethod
    def of(cls, scheme) -> "NativeScheme":
        key = (scheme.name, scheme.a, scheme.b, scheme.c, scheme.clear)
        got = cls._cache.get(key)
        if got is None:
            got = cls._cache[key] = cls(scheme)
        return got

    def plan(self):
        """The native epilogue plan as ``[[(bi, bj, coeff, is_first), ...] per step]``."""
        buf = (ctypes.c_int8 * (16 * 7))()
        counts = (ctypes.c_int32 * 7)()
        check(lib().lcg_scheme_plan(self.handle, buf, counts))
        return [[(buf[t * 16 + 4 * n], buf[t * 16 + 4 * n + 1], buf[t * 16 + 4 * n + 2],
                  bool(buf[t * 16 + 4 * n + 3])) for n in range(counts[t])]
                for t in range(self.scheme.rank)]


def plane_geometry(rows: int, cols: int, row_align: int):
    r2, k2, k2p = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    check(lib().lcg_plane_geometry(rows, cols, row_align, ctypes.byref(r2), ctypes.byref(k2),
                                   ctypes.byref(k2p)))
    return r2.value, k2.value, k2p.value


def stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return t.data_ptr() if t is not None else 0
