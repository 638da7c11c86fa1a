"""Kind table of the batched GEMM: mirror of `frink_cuda::mul_mm`
(crates/frink-cuda/src/mul_mm.rs `KINDS`, `kind_by_name`, `worth_a_gemm` :634)."""
from .matvec_kinds import KINDS as _MV, MatvecKind as MulMmKind, kind_by_name as _by_name  # noqa: F401

KINDS = _MV  # the matvec table and the GEMM table name the same kinds
GEMV_MAX_BATCH = 8


def kind_by_name(name):
    return _by_name(name)


def worth_a_gemm(batch):
    """Below this a batch goes through the GEMV (weights are still read once for
    the whole batch); from it up, through the tensor-core GEMM."""
    return batch > GEMV_MAX_BATCH
