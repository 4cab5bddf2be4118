"""Architecture detection, as the reference's ``pyptx._arch.detect_arch`` (pyptx/_arch.py:1-84)."""
from __future__ import annotations


def detect_arch(default: str = "sm_100a") -> str:
    """``sm_XYa`` string of CUDA device 0, or ``default`` when no GPU is visible."""
    try:
        import torch
        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability(0)
            suffix = "a" if major >= 9 else ""
            return f"sm_{major}{minor}{suffix}"
    except Exception:  # noqa: BLE001 - detection is best effort
        pass
    return default
