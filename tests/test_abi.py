"""The C-ABI library on a machine without a GPU: it loads, exports every symbol the
public header declares, and its registry / validation logic behaves as documented.
No kernel is launched here."""
import ctypes
import os
import re

import pytest

from pyptx_b200 import _ids, _native
from tests.conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    return _native.load()


def test_header_symbols_are_exported(lib):
    header = open(os.path.join(ROOT, "include", "pyptx_b200.h")).read()
    declared = set(re.findall(r"PB200_API[^;(]*?\b(pb200_\w+)\s*\(", header))
    assert len(declared) >= 13
    assert declared == set(_native.EXPORTED_SYMBOLS)
    for sym in declared:
        assert hasattr(lib, sym), sym


def test_header_constants_match_python_ids():
    header = open(os.path.join(ROOT, "include", "pyptx_b200.h")).read()
    for name, value in re.findall(r"#define PB200_(K_\w+|ERR_\w+)\s+(-?\d+)", header):
        if name == "ERR_LEN":
            assert int(value) == _native.ERR_LEN
        else:
            assert getattr(_ids, name) == int(value), name
    flags = re.findall(r"#define PB200_(F_\w+)\s+\((\d+)ull << (\d+)\)", header)
    assert len(flags) >= 8
    for name, mult, shift in flags:
        assert getattr(_ids, name) == int(mult) << int(shift), name


def test_version_and_arch(lib):
    assert lib.pb200_arch() == b"sm_100a"
    assert re.match(rb"\d+\.\d+\.\d+", lib.pb200_version())


def test_registry_lifecycle(lib):
    n0 = lib.pb200_registry_size()
    h = _native.create_handle(_ids.K_RMS_NORM, (2048, 8192), (1e-6,))
    assert h > 0 and lib.pb200_has_handle(h) == 1 and lib.pb200_registry_size() == n0 + 1
    g = _native.geometry_of(h)
    assert tuple(g.grid) == (2048, 1, 1) and tuple(g.block) == (256, 1, 1) and tuple(g.cluster) == (1, 1, 1)
    assert (g.n_inputs, g.n_outputs) == (2, 1)
    assert lib.pb200_destroy(h) == 0 and lib.pb200_has_handle(h) == 0
    assert lib.pb200_destroy(h) == _ids.ERR_UNKNOWN_HANDLE
    assert lib.pb200_registry_size() == n0


def test_create_rejects_bad_shapes(lib):
    err = ctypes.create_string_buffer(_native.ERR_LEN)

    def create(kid, dims):
        d = (ctypes.c_int64 * len(dims))(*dims)
        return lib.pb200_create(kid, d, len(dims), None, 0, 0, err), err.value.decode()

    rc, msg = create(_ids.K_RMS_NORM, (4, 66))
    assert rc == _ids.ERR_BAD_SHAPE and "divisible by 4" in msg
    rc, msg = create(_ids.K_GEMM_1SM, (100, 256, 64))
    assert rc == _ids.ERR_BAD_SHAPE and "M=100 must be divisible by 128" in msg
    rc, msg = create(_ids.K_GEMM_2SM, (128, 256, 64))
    assert rc == _ids.ERR_BAD_SHAPE and "M=128 must be divisible by 256" in msg
    rc, msg = create(_ids.K_GEMM_1SM, (128, 128, 64))
    assert rc == _ids.ERR_BAD_SHAPE and "N=128 must be divisible by 256" in msg
    rc, msg = create(_ids.K_GEMM_1SM, (128, 256, 96))
    assert rc == _ids.ERR_BAD_SHAPE and "K=96 must be divisible by 64" in msg
    rc, msg = create(_ids.K_GROUPED_GEMM, (2, 128, 32, 64))
    assert rc == _ids.ERR_BAD_SHAPE and "N=32" in msg
    rc, msg = create(99, (1, 1))
    assert rc == _ids.ERR_BAD_KERNEL
    rc, msg = create(_ids.K_SOFTMAX, (1, 2, 3))
    assert rc == _ids.ERR_BAD_SHAPE


def test_gemm_geometry(lib):
    h = _native.create_handle(_ids.K_GEMM_1SM, (8192, 8192, 8192))
    g = _native.geometry_of(h)
    assert tuple(g.block) == (192, 1, 1) and tuple(g.cluster) == (1, 1, 1)
    assert g.grid[0] <= 148 or g.grid[0] % 2 == 0
    assert 200 * 1024 < g.smem_bytes <= 227 * 1024
    h2 = _native.create_handle(_ids.K_GEMM_2SM, (8192, 8192, 8192))
    g2 = _native.geometry_of(h2)
    assert tuple(g2.cluster) == (2, 1, 1) and g2.grid[0] % 2 == 0
    h3 = _native.create_handle(_ids.K_GROUPED_GEMM, (8, 2048, 256, 2048))
    assert _native.geometry_of(h3).grid[0] == min(128, _native.geometry_of(h).grid[0])
    for x in (h, h2, h3):
        lib.pb200_destroy(x)


def test_launch_validation_happens_before_any_cuda_call(lib):
    err = ctypes.create_string_buffer(_native.ERR_LEN)
    ptrs = (ctypes.c_void_p * 3)(0x1000, 0x2000, 0x3000)
    assert lib.pb200_launch_raw(10**9, 0, ptrs, 3, err) == _ids.ERR_UNKNOWN_HANDLE
    assert b"unknown handle" in err.value
    h = _native.create_handle(_ids.K_RMS_NORM, (4, 64), (1e-6,))
    assert lib.pb200_launch_raw(h, 0, ptrs, 2, err) == _ids.ERR_ARG_COUNT
    assert b"takes 3 buffers" in err.value
    bad = (ctypes.c_void_p * 3)(0x1000, 0x2004, 0x3000)
    assert lib.pb200_launch_raw(h, 0, bad, 3, err) == _ids.ERR_MISALIGNED
    assert b"buffer 1" in err.value
    null = (ctypes.c_void_p * 3)(0x1000, 0, 0x3000)
    assert lib.pb200_launch_raw(h, 0, null, 3, err) == _ids.ERR_MISALIGNED
    assert lib.pb200_launch_raw(h, 0, ptrs, 3, None) != 0 or True  # NULL err_out is accepted
    lib.pb200_destroy(h)


def test_encodings_match_oracle(lib):
    from oracle import encodings
    for m in (64, 128, 256):
        for n in (64, 128, 256):
            for am in (0, 1):
                for bm in (0, 1):
                    want = encodings.instr_desc_f16bf16_f32(m=m, n=n, a_major="MN" if am else "K",
                                                            b_major="MN" if bm else "K")
                    assert lib.pb200_encode_idesc(m, n, 1, am, bm) == want
    assert lib.pb200_encode_idesc(128, 256, 0, 0, 0) == 0x08400010
    assert lib.pb200_encode_smem_desc(0, 16, 1024, 2) == encodings.SMEM_DESC_SW128_KMAJOR
    for addr in (0x400, 0x12340, 0x3FFF0):
        assert lib.pb200_encode_smem_desc(addr, 16, 1024, 2) == encodings.smem_desc(addr, stride_bytes=1024)
        assert lib.pb200_encode_smem_desc(addr, 16384, 1024, 2) == encodings.smem_desc(
            addr, stride_bytes=1024, leading_bytes=16384)
    for off in range(0, 4096, 16):
        assert lib.pb200_swizzle128(off) == encodings.swizzle_128b(off)


def test_push_gemm_and_peer_barrier_geometry(lib):
    err = ctypes.create_string_buffer(_native.ERR_LEN)

    def create(kid, dims, fparams=()):
        d = (ctypes.c_int64 * len(dims))(*dims)
        f = (ctypes.c_double * max(len(fparams), 1))(*fparams)
        return lib.pb200_create(kid, d, len(dims), f, len(fparams), 0, err), err.value.decode()

    h = _native.create_handle(_ids.K_GEMM_PUSH, (4, 2, 1024, 512, 256))
    g = _native.geometry_of(h)
    assert (g.n_inputs, g.n_outputs) == (2, 4) and tuple(g.cluster) == (2, 1, 1) and g.scratch_bytes == 0
    h1 = _native.create_handle(_ids.K_GEMM_PUSH, (1, 1, 128, 256, 64))
    g1 = _native.geometry_of(h1)
    assert (g1.n_inputs, g1.n_outputs) == (2, 1) and tuple(g1.cluster) == (1, 1, 1)
    rc, msg = create(_ids.K_GEMM_PUSH, (9, 2, 1024, 512, 256))
    assert rc == _ids.ERR_BAD_SHAPE and "destination count" in msg
    rc, msg = create(_ids.K_GEMM_PUSH, (2, 3, 1024, 512, 256))
    assert rc == _ids.ERR_BAD_SHAPE and "cta_group" in msg
    rc, msg = create(_ids.K_GEMM_PUSH, (2, 2, 128, 512, 256))
    assert rc == _ids.ERR_BAD_SHAPE and "M=128 must be divisible by 256" in msg
    rc, msg = create(_ids.K_GEMM_PUSH, (1024, 512, 256))
    assert rc == _ids.ERR_BAD_SHAPE

    hb = _native.create_handle(_ids.K_PEER_BARRIER, (8, 3))
    gb = _native.geometry_of(hb)
    assert (gb.n_inputs, gb.n_outputs) == (8, 0) and tuple(gb.grid) == (1, 1, 1) and tuple(gb.block) == (32, 1, 1)
    rc, msg = create(_ids.K_PEER_BARRIER, (9, 0))
    assert rc == _ids.ERR_BAD_SHAPE and "world" in msg
    rc, msg = create(_ids.K_PEER_BARRIER, (2, 2))
    assert rc == _ids.ERR_BAD_SHAPE and "rank" in msg
    rc, msg = create(_ids.K_PEER_BARRIER, (2, 0), (0.0,))
    assert rc == _ids.ERR_BAD_SHAPE and "timeout" in msg
    for x in (h, h1, hb):
        lib.pb200_destroy(x)


def test_registry_is_safe_under_concurrent_use(lib):
    """The registry is shared by every thread of the host process (the reference guards its own
    with one mutex, pyptx/_shim/pyptx_launch.cc:236-237): concurrent create / query / destroy
    must neither lose nor duplicate handles, and each call reports through its own buffer."""
    import threading

    before = lib.pb200_registry_size()
    per_thread, n_threads = 200, 8
    handles: list[list[int]] = [[] for _ in range(n_threads)]
    errors: list[str] = []

    def worker(i: int) -> None:
        err = ctypes.create_string_buffer(_native.ERR_LEN)
        try:
            for j in range(per_thread):
                d = (ctypes.c_int64 * 2)(4 + i, 64 * (1 + j % 4))
                f = (ctypes.c_double * 1)(1e-6)
                h = lib.pb200_create(_ids.K_RMS_NORM, d, 2, f, 1, 0, err)
                if h <= 0 or not lib.pb200_has_handle(h):
                    errors.append(f"thread {i}: create -> {h} {err.value!r}")
                    return
                g = _native.Geometry()
                if lib.pb200_geometry_of(h, ctypes.byref(g)) != 0 or g.grid[0] != 4 + i:
                    errors.append(f"thread {i}: geometry of {h} is another thread's")
                    return
                handles[i].append(h)
                bad = (ctypes.c_int64 * 2)(4, 66)
                if lib.pb200_create(_ids.K_RMS_NORM, bad, 2, f, 1, 0, err) != _ids.ERR_BAD_SHAPE or b"divisible" not in err.value:
                    errors.append(f"thread {i}: rejection message got mixed up: {err.value!r}")
                    return
                if j % 3 == 2:
                    lib.pb200_destroy(handles[i].pop(0))
        except Exception as exc:  # noqa: BLE001
            errors.append(f"thread {i}: {exc!r}")

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(n_threads)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]
    live = [h for hs in handles for h in hs]
    assert len(set(live)) == len(live)
    assert lib.pb200_registry_size() == before + len(live)
    for h in live:
        assert lib.pb200_has_handle(h)
        lib.pb200_destroy(h)
    assert lib.pb200_registry_size() == before


def test_attention_backward_geometry(lib):
    """Scratch of the attention backward handle: delta and lse*log2(e) per padded query, plus (fused
    form only) the fp32 dQ accumulator with rows of the tile's head dimension."""
    BH, SQ, SKV = 6, 300, 520
    sq_pad = 384
    for hd, tile in ((64, 64), (40, 64), (128, 128), (72, 128)):
        fused = _native.create_handle(_ids.K_FLASH_ATTN_BWD, (BH, SQ, SKV, hd), (0.0,), _ids.F_CAUSAL)
        two_pass = _native.create_handle(_ids.K_FLASH_ATTN_BWD, (BH, SQ, SKV, hd), (0.0,),
                                         _ids.F_CAUSAL | _ids.F_DETERMINISTIC)
        gf, gt = _native.geometry_of(fused), _native.geometry_of(two_pass)
        assert (gf.n_inputs, gf.n_outputs) == (6, 3) == (gt.n_inputs, gt.n_outputs)
        assert gt.scratch_bytes == 2 * BH * sq_pad * 4
        assert gf.scratch_bytes == gt.scratch_bytes + BH * sq_pad * tile * 4
        assert tuple(gf.grid) == ((SKV + 127) // 128, BH, 1) and tuple(gf.block) == (384, 1, 1)
        assert gf.smem_bytes <= 227 * 1024 and gt.smem_bytes <= 227 * 1024
        lib.pb200_destroy(fused)
        lib.pb200_destroy(two_pass)
