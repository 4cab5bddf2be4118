"""Builds and loads the C-ABI library (``libpyptx_b200.so``).

Counterpart of the reference's shim loader and auto-build
(pyptx/jax_support.py:132-230 ``_load_shim``; pyptx/_shim/auto_build.py:20-69):
the library is compiled in-tree with ``nvcc`` for ``sm_100a`` and opened with
``ctypes``.  There is no CPU fallback: if the library cannot be built or loaded,
every kernel call raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(_PKG_DIR, "csrc")
INCLUDE_DIR = os.path.join(os.path.dirname(_PKG_DIR), "include")
LIB_DIR = os.path.join(_PKG_DIR, "_lib")
# PYPTX_B200_LIB points at a library built elsewhere (e.g. an installed copy); default: in-tree.
LIB_PATH = os.environ.get("PYPTX_B200_LIB") or os.path.join(LIB_DIR, "libpyptx_b200.so")

ERR_LEN = 128

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-shared",
]

# Every symbol include/pyptx_b200.h declares.
EXPORTED_SYMBOLS = (
    "pb200_create", "pb200_launch_raw", "pb200_geometry_of", "pb200_has_handle",
    "pb200_registry_size", "pb200_clear_registry", "pb200_destroy",
    "pb200_device_status", "pb200_version", "pb200_arch",
    "pb200_encode_idesc", "pb200_encode_smem_desc", "pb200_swizzle128",
    "pb200_rms_norm_bwd_static",
)


class Geometry(ctypes.Structure):
    """Mirror of ``pb200_geometry`` in include/pyptx_b200.h."""

    _fields_ = [
        ("grid", ctypes.c_uint32 * 3),
        ("block", ctypes.c_uint32 * 3),
        ("cluster", ctypes.c_uint32 * 3),
        ("smem_bytes", ctypes.c_uint32),
        ("n_inputs", ctypes.c_uint32),
        ("n_outputs", ctypes.c_uint32),
        ("scratch_bytes", ctypes.c_uint64),
    ]


def cuda_sources() -> list[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _all_sources() -> list[str]:
    deps = [os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR)
            if f.endswith((".cu", ".cuh", ".h"))]
    deps += [os.path.join(INCLUDE_DIR, f) for f in os.listdir(INCLUDE_DIR) if f.endswith(".h")]
    return deps


def is_stale() -> bool:
    if not os.path.isfile(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in _all_sources())


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """Compile every ``csrc/*.cu`` into ``_lib/libpyptx_b200.so``.

    Object files are cached under ``_lib/obj`` and rebuilt when a source or
    header is newer.  Returns the library path.
    """
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("pyptx_b200: nvcc not found; cannot build " + LIB_PATH)
    if not force and not is_stale():
        return LIB_PATH
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    headers = [p for p in _all_sources() if not p.endswith(".cu")]
    newest_header = max(os.path.getmtime(p) for p in headers)
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]
    if ptxas_info:
        compile_flags += ["-Xptxas", "-v"]
    jobs = []
    objs = []
    for src in cuda_sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if (force or not os.path.isfile(obj) or os.path.getmtime(obj) < os.path.getmtime(src)
                or os.path.getmtime(obj) < newest_header):
            cmd = [nvcc, *compile_flags, "-I", INCLUDE_DIR, "-c", src, "-o", obj]
            jobs.append((src, cmd))
    results: dict[str, subprocess.CompletedProcess] = {}

    def run(src, cmd):
        results[src] = subprocess.run(cmd, capture_output=True, text=True)

    threads = [threading.Thread(target=run, args=j) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for src, cmd in jobs:
        r = results[src]
        if verbose or ptxas_info or r.returncode != 0:
            print(" ".join(cmd))
            print(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"pyptx_b200: nvcc failed on {src}:\n{r.stderr}")
    tmp = LIB_PATH + ".tmp"
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC", "-o", tmp, *objs]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"pyptx_b200: link failed:\n{r.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


TORCH_EXT_NAME = "_pb200_torch_ext"
TORCH_EXT_PATH = os.path.join(LIB_DIR, TORCH_EXT_NAME + ".so")
TORCH_EXT_SRC = os.path.join(CSRC_DIR, "torch_ext.cpp")


def build_torch_ext(force: bool = False) -> str:
    """Compile ``csrc/torch_ext.cpp`` (pybind11 fast path) in-tree with g++ against the installed
    torch; counterpart of the reference's JIT build of its extension
    (pyptx/torch_support.py:128-149), done ahead of time so that it travels with the tree."""
    if (not force and os.path.isfile(TORCH_EXT_PATH)
            and os.path.getmtime(TORCH_EXT_PATH) >= os.path.getmtime(TORCH_EXT_SRC)):
        return TORCH_EXT_PATH
    import sysconfig
    import warnings

    import torch
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        from torch.utils import cpp_extension as ce
        inc, libdirs = ce.include_paths(), ce.library_paths()
    os.makedirs(LIB_DIR, exist_ok=True)
    tmp = TORCH_EXT_PATH + ".tmp"
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", TORCH_EXT_SRC, "-o", tmp,
           f"-DTORCH_EXTENSION_NAME={TORCH_EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I" + sysconfig.get_paths()["include"]]
    cmd += ["-I" + i for i in inc if os.path.isdir(i) and "cuda" not in i]
    libdirs = [d for d in libdirs if os.path.isdir(d) and "cuda" not in d]
    cmd += ["-L" + d for d in libdirs]
    cmd += ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-ldl"]
    cmd += ["-Wl,-rpath," + d for d in libdirs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"pyptx_b200: building the torch extension failed:\n{r.stderr[-2000:]}")
    os.replace(tmp, TORCH_EXT_PATH)
    return TORCH_EXT_PATH


_TORCH_EXT = None
_TORCH_EXT_TRIED = False


def load_torch_ext():
    """The pybind11 extension module with the C-ABI library attached, or ``None`` when it has
    not been built (the ctypes path is then used; both end in the same ``pb200_launch_raw``).
    ``PYPTX_B200_NO_TORCH_EXT=1`` forces the ctypes path."""
    global _TORCH_EXT, _TORCH_EXT_TRIED
    if _TORCH_EXT_TRIED:
        return _TORCH_EXT
    with _LOCK:
        if _TORCH_EXT_TRIED:
            return _TORCH_EXT
        ext = None
        if os.environ.get("PYPTX_B200_NO_TORCH_EXT") != "1" and os.path.isfile(TORCH_EXT_PATH):
            import importlib.util

            import torch  # noqa: F401 - libtorch must be loaded before the extension
            try:
                spec = importlib.util.spec_from_file_location(TORCH_EXT_NAME, TORCH_EXT_PATH)
                ext = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(ext)
                ext.load_shim(LIB_PATH)
            except Exception:  # noqa: BLE001 - an unusable extension falls back to ctypes, same C ABI
                ext = None
        _TORCH_EXT = ext
        _TORCH_EXT_TRIED = True
    return _TORCH_EXT


_LIB = None
_LOCK = threading.Lock()


def load():
    """Return the loaded library with ctypes signatures attached.

    Builds it first when it is missing and ``nvcc`` is present.  Raises
    ``RuntimeError`` otherwise -- callers must not degrade to another path.
    """
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        if not os.path.isfile(LIB_PATH):
            try:
                build()
            except Exception as exc:  # noqa: BLE001 - reported with context below
                raise RuntimeError(
                    f"pyptx_b200: native library {LIB_PATH} is missing and could not be built "
                    f"({exc}). Run `python -m pyptx_b200.build`.") from exc
        try:
            lib = ctypes.CDLL(LIB_PATH)
        except OSError as exc:
            raise RuntimeError(f"pyptx_b200: cannot load {LIB_PATH}: {exc}") from exc
        for sym in EXPORTED_SYMBOLS:
            if not hasattr(lib, sym):
                raise RuntimeError(f"pyptx_b200: {LIB_PATH} does not export {sym}; rebuild it")
        c = ctypes
        lib.pb200_create.restype = c.c_int64
        lib.pb200_create.argtypes = [c.c_int32, c.POINTER(c.c_int64), c.c_size_t,
                                     c.POINTER(c.c_double), c.c_size_t, c.c_uint64, c.c_char_p]
        lib.pb200_launch_raw.restype = c.c_int
        lib.pb200_launch_raw.argtypes = [c.c_int64, c.c_uint64, c.c_void_p, c.c_size_t, c.c_char_p]
        lib.pb200_geometry_of.restype = c.c_int
        lib.pb200_geometry_of.argtypes = [c.c_int64, c.POINTER(Geometry)]
        lib.pb200_has_handle.restype = c.c_int
        lib.pb200_has_handle.argtypes = [c.c_int64]
        lib.pb200_registry_size.restype = c.c_size_t
        lib.pb200_registry_size.argtypes = []
        lib.pb200_clear_registry.restype = None
        lib.pb200_clear_registry.argtypes = []
        lib.pb200_destroy.restype = c.c_int
        lib.pb200_destroy.argtypes = [c.c_int64]
        lib.pb200_device_status.restype = c.c_int
        lib.pb200_device_status.argtypes = [c.c_char_p]
        lib.pb200_version.restype = c.c_char_p
        lib.pb200_version.argtypes = []
        lib.pb200_arch.restype = c.c_char_p
        lib.pb200_arch.argtypes = []
        lib.pb200_encode_idesc.restype = c.c_uint32
        lib.pb200_encode_idesc.argtypes = [c.c_int32] * 5
        lib.pb200_encode_smem_desc.restype = c.c_uint64
        lib.pb200_encode_smem_desc.argtypes = [c.c_uint32] * 4
        lib.pb200_swizzle128.restype = c.c_uint32
        lib.pb200_swizzle128.argtypes = [c.c_uint32]
        lib.pb200_rms_norm_bwd_static.restype = c.c_int
        lib.pb200_rms_norm_bwd_static.argtypes = [c.c_int64, c.c_int64, c.c_double, c.c_uint64, c.c_void_p, c.c_void_p,
                                                  c.c_void_p, c.c_void_p, c.c_void_p, c.c_char_p]
        _LIB = lib
    return _LIB


def create_handle(kernel_id: int, dims, fparams=(), flags: int = 0) -> int:
    """``pb200_create`` with Python sequences; raises ``ValueError`` on rejection."""
    lib = load()
    d = (ctypes.c_int64 * max(len(dims), 1))(*[int(x) for x in dims])
    f = (ctypes.c_double * max(len(fparams), 1))(*[float(x) for x in fparams])
    err = ctypes.create_string_buffer(ERR_LEN)
    h = lib.pb200_create(kernel_id, d, len(dims), f, len(fparams), flags, err)
    if h <= 0:
        raise ValueError(f"pyptx_b200: pb200_create failed (code {h}): {err.value.decode(errors='replace')}")
    return int(h)


def launch_raw(handle: int, stream: int, ptrs) -> None:
    """``pb200_launch_raw`` on raw device addresses (``ptrs``: ints, or a prepared
    ``c_void_p`` array); raises ``RuntimeError`` with the library's message on failure."""
    lib = load()
    if not isinstance(ptrs, ctypes.Array):
        ptrs = (ctypes.c_void_p * len(ptrs))(*[int(x) for x in ptrs])
    err = ctypes.create_string_buffer(ERR_LEN)
    rc = lib.pb200_launch_raw(handle, int(stream), ctypes.cast(ptrs, ctypes.c_void_p), len(ptrs), err)
    if rc != 0:
        raise RuntimeError(f"pyptx_b200: pb200_launch_raw failed (code {rc}): {err.value.decode(errors='replace')}")


def geometry_of(handle: int) -> Geometry:
    g = Geometry()
    rc = load().pb200_geometry_of(handle, ctypes.byref(g))
    if rc != 0:
        raise RuntimeError(f"pyptx_b200: pb200_geometry_of failed (code {rc})")
    return g


def device_status() -> None:
    """Synchronise and raise if a bounded device-side wait gave up."""
    err = ctypes.create_string_buffer(ERR_LEN)
    rc = load().pb200_device_status(err)
    if rc != 0:
        raise RuntimeError(f"pyptx_b200: device status (code {rc}): {err.value.decode(errors='replace')}")
