"""Integer encodings on the tcgen05 path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Plain-Python restatements of the bit layouts the reference encodes; the CUDA
side has its own copy in ``pyptx_b200/csrc/ptx.cuh`` and tests compare the two.
"""
from __future__ import annotations

_MAJOR = {"K": 0, "MN": 1}
_AB_FORMAT = {"f16": 0, "bf16": 1, "tf32": 2}
_LAYOUT = {"NONE": 0, "128B_BASE32B": 1, "128B": 2, "64B": 4, "32B": 6}

# pyptx/ptx.py:3399-3405 with LBO 16, SBO 1024, version 1, 128-byte swizzle;
# the constant the reference's GEMMs use (gemm_highperf_blackwell.py:50) and its
# tests pin (tests/test_typed_wrappers.py:427-438).
SMEM_DESC_SW128_KMAJOR = 0x4000404000010000


def instr_desc_f16bf16_f32(*, m: int = 128, n: int = 256, ab_dtype: str = "bf16", a_major: str = "K",
                           b_major: str = "K", scale_a: int = 1, scale_b: int = 1,
                           saturate: bool = False, sparse: bool = False, max_shift: int = 0) -> int:
    """32-bit tcgen05 instruction descriptor, f16/bf16/tf32 inputs, f32 accumulate
    (pyptx/ptx.py:3312-3366)."""
    if m not in (64, 128, 256):
        raise ValueError("m must be 64, 128, or 256")
    if n % 8 != 0 or not 8 <= n <= 256:
        raise ValueError("n must be a multiple of 8 between 8 and 256")
    if scale_a not in (1, -1) or scale_b not in (1, -1):
        raise ValueError("scale must be 1 or -1")
    fmt = _AB_FORMAT[ab_dtype]
    d = 0
    d |= int(bool(sparse)) << 2
    d |= int(bool(saturate)) << 3
    d |= 1 << 4
    d |= fmt << 7
    d |= fmt << 10
    d |= (0 if scale_a == 1 else 1) << 13
    d |= (0 if scale_b == 1 else 1) << 14
    d |= _MAJOR[a_major] << 15
    d |= _MAJOR[b_major] << 16
    d |= (n >> 3) << 17
    d |= (m >> 4) << 24
    d |= max_shift << 30
    return d


def smem_desc(smem_addr: int, *, stride_bytes: int, leading_bytes: int = 16, swizzle: str = "128B",
              version: int = 1, base_offset: int = 0, lbo_mode: int = 0) -> int:
    """64-bit shared-memory matrix descriptor (pyptx/ptx.py:3368-3459): start address,
    leading / stride byte offsets (all >> 4), version, base offset, LBO mode, layout."""
    if stride_bytes % 16 or leading_bytes % 16:
        raise ValueError("byte offsets must be multiples of 16")
    d = (smem_addr >> 4) & 0x3FFF
    d |= (leading_bytes >> 4) << 16
    d |= (stride_bytes >> 4) << 32
    d |= version << 46
    d |= base_offset << 49
    d |= lbo_mode << 52
    d |= _LAYOUT[swizzle] << 61
    return d


def swizzle_128b(offset: int) -> int:
    """Swizzle<3,4,3>: ``phys = off ^ ((off & 0x380) >> 3)`` (pyptx/smem.py:476-492)."""
    return offset ^ ((offset & 0x380) >> 3)


def swizzle(offset: int, kind: str | None) -> int:
    """32B / 64B / 128B swizzles of pyptx/smem.py:488-492; ``None`` is the identity."""
    if kind is None:
        return offset
    mask = {"32B": 0x080, "64B": 0x180, "128B": 0x380}[kind]
    return offset ^ ((offset & mask) >> 3)
