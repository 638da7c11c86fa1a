"""Kind table of the decode matvecs: mirror of `frink_cuda::matvec_kinds`
(crates/frink-cuda/src/matvec_kinds.rs `KINDS`, `kind_by_name`; the dp4a table
crates/frink-cuda/src/matvec_kinds/dp4a.rs:201-242)."""
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class MatvecKind:
    name: str          # QuantKind name as frink-core spells it
    fn_name: str       # the frink-cuda entry this library's kernel stands in for
    tag: int           # ggml type tag = fk_kind
    block_bytes: int
    block_elems: int


KINDS = (
    MatvecKind("Q4_K", "q4_k_matvec", 12, 144, 256),
    MatvecKind("Q5_K", "q5_k_matvec", 13, 176, 256),
    MatvecKind("Q6_K", "q6_k_matvec", 14, 210, 256),
    MatvecKind("Q8_0", "q8_0_matvec", 8, 34, 32),
    MatvecKind("MXFP4", "mxfp4_matvec", 39, 17, 32),
)


def kind_by_name(name):
    """By QuantKind name or by frink-cuda kernel name; None for a kind with no kernel here."""
    key = str(name).lower()
    for k in KINDS:
        if key in (k.name.lower(), k.fn_name, k.fn_name + "_dp4a"):
            return k
    return None


def kind_by_tag(tag):
    for k in KINDS:
        if k.tag == int(tag):
            return k
    return None


def matvec_reads(fn_name, n_blocks, x):
    """What a decode matvec reads of `x`: its q8_1 rounding, per run of 32
    (`matvec_kinds::dp4a::matvec_reads`, dp4a.rs:291-303).  Every kind in KINDS
    quantizes; an input that is not whole runs is refused, not passed through."""
    from . import device
    x = np.ascontiguousarray(x, np.float32)
    if kind_by_name(fn_name) is None or x.size % 32:
        return x.copy()
    y = device.quantize_q8_1_host(x).reshape(-1, 36)
    d = y[:, :2].copy().view(np.float16).astype(np.float32)
    return (y[:, 4:].view(np.int8).astype(np.float32) * d).reshape(x.shape)
