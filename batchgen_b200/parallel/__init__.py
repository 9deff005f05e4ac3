"""Multi-GPU layer: symmetric heap over NVLink, fused compute+collective kernels, NCCL baselines."""


def make_comm(kind: str = "auto", device=None):
    """``fused`` = in-kernel NVLink communication (falls back to NCCL only when ``auto`` and the
    symmetric heap cannot be set up); ``nccl`` = the baseline collectives."""
    from .comm import NcclComm
    if kind in ("auto", "fused"):
        try:
            from .fused import FusedComm
            return FusedComm(device=device)
        except Exception:
            if kind == "fused":
                raise
    return NcclComm()
