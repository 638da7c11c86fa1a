"""Kind table of the prefill GEMM: mirror of `frink_cuda::mul_mm`
(crates/frink-cuda/src/mul_mm.rs `KINDS`, `kind_by_name`, `worth_a_gemm` :634)."""
from .matvec_kinds import KINDS as _MV, MatvecKind as MulMmKind, kind_by_name as _by_name  # noqa: F401

KINDS = tuple(k for k in _MV if k.name != "Q5_K")   # every matvec kind but Q5_K, which has the plain matvec only
GEMV_MAX_BATCH = 8


def kind_by_name(name):
    k = _by_name(name)
    return k if k in KINDS else None


def worth_a_gemm(batch):
    """Below this a batch goes through the GEMV (weights are still read once for
    the whole batch); from it up, through the tensor-core GEMM."""
    return batch > GEMV_MAX_BATCH
