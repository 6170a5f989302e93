"""CPU oracle for the OrthoLinear forward.  TEST INFRASTRUCTURE ONLY.

Two checkers live here, both reached through ``ctypes``:

* ``impl="port"``       -- ``liboracle.so``: this repository's plain-C restatement of the
  reference CPU forward (``ortho_oracle.c``; follows ``src/ortho.c:315-402``).
* ``impl="reference"``  -- ``_ref/libortho_ref.so``: the reference's own unmodified
  ``src/ortho.c`` behind ``ref_harness.c`` (row-chunked calls, strict FP32 order).
  ``impl="reference_fast"`` is the same code built with the reference's own flags
  (``tests/Makefile:4``) and is what the benchmark times.

Only the test-suite, the smoke entry and the benchmark's CPU legs may import this package;
the shipped library (``libortho_b200``) never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS: dict = {}

_PATHS = {
    "port": os.path.join(_HERE, "liboracle.so"),
    "reference": os.path.join(_HERE, "_ref", "libortho_ref.so"),
    "reference_fast": os.path.join(_HERE, "_ref", "libortho_ref_fast.so"),
}


def reference_root():
    """Where the reference's source tree lies: ``$LIBORTHO_REF``, else a ``reference`` directory
    beside this repository; None when neither holds ``src/ortho.c``."""
    cands = [os.environ.get("LIBORTHO_REF"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "src", "ortho.c")):
            return os.path.abspath(c)
    return None


def build(ref_root=None, quiet: bool = True) -> None:
    """Compile the checker libraries (``make -C oracle``).  The ``_ref`` libraries are only
    rebuilt when the reference tree is found (``ref_root`` or ``reference_root()``); otherwise the
    prebuilt files are kept."""
    ref_root = ref_root or reference_root() or ""
    out = subprocess.run(["make", "-C", _HERE, f"REF={ref_root}", "all"],
                         capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)
    _LIBS.clear()


def available(impl: str) -> bool:
    return os.path.exists(_PATHS[impl])


def _lib(impl: str):
    if impl in _LIBS:
        return _LIBS[impl]
    path = _PATHS[impl]
    if not os.path.exists(path):
        if impl == "port":
            build()
        if not os.path.exists(path):
            raise FileNotFoundError(f"oracle library {path} not built (run `make -C oracle`)")
    lib = ctypes.CDLL(path)
    c = ctypes
    vp = c.c_void_p
    pre = "oracle" if impl == "port" else "ref"
    f = getattr(lib, f"{pre}_forward_csr")
    f.restype = c.c_int
    f.argtypes = [vp, vp, vp, vp, vp, c.c_int64, vp, vp, c.c_size_t, c.c_size_t, c.c_size_t,
                  c.c_float, c.c_int]
    g = getattr(lib, f"{pre}_forward_coo16")
    g.restype = c.c_int
    g.argtypes = [vp, vp, vp, vp, c.c_int, vp, vp, c.c_size_t, c.c_size_t, c.c_size_t, c.c_float]
    if impl == "port":
        lib.oracle_dequant.restype = c.c_int
        lib.oracle_dequant.argtypes = [vp, vp, c.c_size_t, c.c_size_t, vp, vp]
        lib.oracle_unpack_int4.restype = c.c_int8
        lib.oracle_unpack_int4.argtypes = [vp, c.c_size_t]
    else:
        lib.ref_lifecycle_check.restype = c.c_int
        lib.ref_lifecycle_check.argtypes = [c.c_size_t, c.c_size_t, c.c_size_t]
    _LIBS[impl] = lib
    return lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def forward_csr(packed, scales, row_ptr, col, vals, x, alpha, *, impl="port", threads=None):
    """Y[M,N] (float32) for packed INT4 ``packed`` u8 [N,K/2], FP32 ``scales`` [N], CSR ortho
    (``row_ptr`` i32 [N+1], ``col`` i32 [nnz], ``vals`` f32 [nnz]; all three may be ``None``
    for an empty ortho) and FP32 ``x`` [M,K].  FP16 module buffers must be up-cast exactly to
    FP32 by the caller, which is what the reference's all-FP32 C API expects
    (``include/ortho.h:132-135``)."""
    packed = _c(packed, np.uint8)
    N, kh = packed.shape
    K = kh * 2
    scales = _c(scales, np.float32)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    nnz = 0
    if vals is not None and len(vals):
        row_ptr = _c(row_ptr, np.int32)
        col = _c(col, np.int32)
        vals = _c(vals, np.float32)
        nnz = int(vals.shape[0])
        assert row_ptr.shape[0] == N + 1 and col.shape[0] == nnz
    else:
        row_ptr = col = vals = None
    y = np.empty((M, N), dtype=np.float32)
    threads = host_threads() if threads is None else int(threads)
    rc = getattr(_lib(impl), ("oracle" if impl == "port" else "ref") + "_forward_csr")(
        _p(packed), _p(scales), _p(row_ptr), _p(col), _p(vals), nnz, _p(x), _p(y),
        M, K, N, float(alpha), threads)
    if rc != 0:
        raise RuntimeError(f"oracle forward ({impl}) returned {rc}")
    return y


def forward_coo16(packed, scales, flat_idx, vals, x, alpha, *, impl="port"):
    """Forward with the legacy 16-bit coordinate list, in list order, duplicates allowed --
    the exact input form of ``src/ortho.c:384-398`` and of the reference's known-answer test."""
    packed = _c(packed, np.uint8)
    N, kh = packed.shape
    K = kh * 2
    scales = _c(scales, np.float32)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    flat_idx = _c(flat_idx, np.uint16)
    vals = _c(vals, np.float32)
    count = 0 if flat_idx is None else int(flat_idx.shape[0])
    y = np.empty((M, N), dtype=np.float32)
    rc = getattr(_lib(impl), ("oracle" if impl == "port" else "ref") + "_forward_coo16")(
        _p(packed), _p(scales), _p(flat_idx), _p(vals), count, _p(x), _p(y), M, K, N, float(alpha))
    if rc != 0:
        raise RuntimeError(f"oracle coo16 forward ({impl}) returned {rc}")
    return y


def dequant(packed, scales):
    """(w_int int8 [N,K], w_deq float32 [N,K]) following ``src/ortho.c:315-325,363``."""
    packed = _c(packed, np.uint8)
    N, kh = packed.shape
    K = kh * 2
    scales = _c(scales, np.float32)
    wi = np.empty((N, K), dtype=np.int8)
    wd = np.empty((N, K), dtype=np.float32)
    rc = _lib("port").oracle_dequant(_p(packed), _p(scales), N, K, _p(wi), _p(wd))
    if rc != 0:
        raise RuntimeError("oracle_dequant failed")
    return wi, wd


def unpack_int4_numpy(packed):
    """Vectorised numpy statement of the nibble rule of ``src/ortho.c:315-325`` (low nibble =
    even element, 4-bit two's complement); cross-checks the C restatement in the tests."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    lo = (packed & 0x0F).astype(np.int16)
    hi = (packed >> 4).astype(np.int16)
    lo = lo - ((lo & 8) << 1)
    hi = hi - ((hi & 8) << 1)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.int8)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


def lifecycle_check(K: int, N: int, nnz: int) -> int:
    return int(_lib("reference").ref_lifecycle_check(K, N, nnz))
