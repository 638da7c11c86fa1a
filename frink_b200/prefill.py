"""The resident routed (MoE) layer: mirror of `frink_cuda::prefill::moe_device`
(crates/frink-cuda/src/prefill/moe_device.rs:241-318 `run_device_routed`, decode;
:320-438 `run_device_routed_batch` + :463-519 `grouped_proj`, prefill).

Everything stays on the device: router logits -> top-k -> (prefill) expert
permutation -> gate, up -> gated activation -> down -> weighted combine in
routing order.  `ops` is the set of device calls (`frink_b200.device` by default);
the multi-GPU layer in `parallel.py` reuses these functions with sharded experts."""
from dataclasses import dataclass
from typing import Any, Optional

SOFTMAX, SOFTMAX_RENORM, SOFTMAX_OVER_CHOSEN = 0, 1, 2   # `DeviceGating`: fk_moe_route modes
SILU, SWIGLU_OAI = 0, 1                                   # `GluCuda`


@dataclass
class RoutedLayer:
    """`ExpertProjCuda` x3 + `RouterCuda` (crates/frink-cuda/src/prefill/mod.rs:73-315):
    stacked expert tensors as one handle each, the f32 router, and the gating."""
    router: Any            # f32 [n_experts, hidden]
    gate: Any              # Weights, n_mats = n_experts, rows = ffn, cols = hidden
    up: Any
    down: Any              # rows = hidden, cols = ffn
    k: int
    mode: int = SOFTMAX_RENORM
    act: int = SILU
    router_bias: Optional[Any] = None
    n_experts: Optional[int] = None

    def __post_init__(self):
        if self.n_experts is None:
            self.n_experts = self.gate.n_mats


def _ops(ops):
    if ops is None:
        from . import device
        return device
    return ops


def route(layer, x, ops=None):
    """Router logits and top-k: ids [batch, k] int32, weights [batch, k] in routing order."""
    ops = _ops(ops)
    if hasattr(ops, "router_route") and (x.dim() == 1 or x.shape[0] <= 8):
        return ops.router_route(layer.router, x, layer.k, layer.mode, layer.router_bias)   # decode: one launch
    logits = ops.router_logits(layer.router, x)
    return ops.moe_route(logits, layer.k, layer.mode, layer.router_bias)


def run_device_routed(layer, x, ops=None, residual=None):
    """Decode: one token `x` [hidden] (or a few, [b, hidden], one after another).
    gate and up are one indexed launch each with the k chosen experts as slots.
    residual (same shape as x): the layer's output is added into it instead of returned."""
    ops = _ops(ops)
    if hasattr(ops, "moe_layer"):
        return ops.moe_layer(layer, x, out=residual, accumulate=residual is not None)     # the whole layer is one C call
    if x.dim() == 2:
        import torch
        if residual is not None:
            for t in range(x.shape[0]):
                run_device_routed(layer, x[t], ops, residual[t])
            return residual
        return torch.stack([run_device_routed(layer, x[t], ops) for t in range(x.shape[0])])
    ids, w = route(layer, x, ops)
    ids1 = ids.reshape(-1)
    g = ops.gemv_multi(layer.gate, ids1, x)
    u = ops.gemv_multi(layer.up, ids1, x)
    if hasattr(ops, "gemv_multi_glu"):
        y = ops.gemv_multi_glu(layer.down, ids1, g, u, layer.act)     # the activation rides in the down projection
    else:
        y = ops.gemv_multi(layer.down, ids1, ops.glu(g, u, layer.act))
    if residual is not None:
        ops.moe_combine(y, None, w, 1, layer.k, out=residual[None] if residual.dim() == 1 else residual, accumulate=True)
        return residual
    return ops.moe_combine(y, None, w, 1, layer.k)[0]


def run_device_routed_rows(layer, x, ops=None, residual=None):
    """Decode of a few independent rows x [b, hidden] (b <= 8) at once: every (row, chosen expert) pair is a slot of
    ONE indexed launch per projection -- b * k slots, the row's activation repeated for its k slots."""
    ops = _ops(ops)
    if hasattr(ops, "moe_layer"):
        return ops.moe_layer(layer, x, out=residual, accumulate=residual is not None)
    b = x.shape[0]
    ids, w = route(layer, x, ops)                         # [b, k]
    ids1 = ids.reshape(-1)
    xr = x.repeat_interleave(layer.k, dim=0)              # slot j reads row j // k
    g = ops.gemv_multi(layer.gate, ids1, xr)
    u = ops.gemv_multi(layer.up, ids1, xr)
    if hasattr(ops, "gemv_multi_glu"):
        y = ops.gemv_multi_glu(layer.down, ids1, g, u, layer.act)
    else:
        y = ops.gemv_multi(layer.down, ids1, ops.glu(g, u, layer.act))
    if residual is not None:
        return ops.moe_combine(y, None, w, b, layer.k, out=residual, accumulate=True)
    return ops.moe_combine(y, None, w, b, layer.k)


def run_device_routed_oai(layer, biases, x, ops=None, residual=None):
    """gpt-oss's routed layer (`run_expert_oai`, crates/frink-moe/src/lib.rs:1039-1060): every expert projection has a
    bias row of its own (biases = (gate_b, up_b, down_b), each [n_experts, rows]) and the activation is the clamped
    SwiGLU (`layer.act` = 1), applied to the BIASED gate and up.  x [b, hidden] -> [b, hidden], or added into
    `residual`.  Up to 8 rows: every (row, expert) pair a slot of the indexed matvecs; more: pairs grouped by expert
    through the grouped GEMMs.  An `ops` with `moe_layer` runs it as one C call (`fk_moe_layer_biased`: the biases
    ride in the matvecs' epilogues); the composition below is what that call does, from the separate entry points."""
    import torch
    ops = _ops(ops)
    if hasattr(ops, "moe_layer"):
        return ops.moe_layer(layer, x, out=residual, accumulate=residual is not None, biases=biases)
    gate_b, up_b, down_b = biases
    b, k = x.shape[0], layer.k
    ids, w = route(layer, x, ops)
    if b <= 8:
        ids1 = ids.reshape(-1)
        xr = x.repeat_interleave(k, dim=0) if b > 1 else x[0]
        g = ops.add_bias_(ops.gemv_multi(layer.gate, ids1, xr), gate_b, ids1)
        u = ops.add_bias_(ops.gemv_multi(layer.up, ids1, xr), up_b, ids1)
        y = ops.add_bias_(ops.gemv_multi_glu(layer.down, ids1, g, u, layer.act), down_b, ids1)
        pair_of = None
    else:
        pairs = b * k
        group_off, gather, pair_of = ops.moe_permute(ids, layer.n_experts)
        # the expert of every permuted row, from the group offsets (no host round trip)
        expert_of = torch.searchsorted(group_off[1:].to(torch.int64), torch.arange(pairs, device=group_off.device), right=True).to(torch.int32)
        g = ops.add_bias_(ops.gemm_grouped(layer.gate, group_off, gather, x, pairs), gate_b, expert_of)
        u = ops.add_bias_(ops.gemm_grouped(layer.up, group_off, gather, x, pairs), up_b, expert_of)
        a = ops.glu(g, u, layer.act)
        y = ops.add_bias_(ops.gemm_grouped(layer.down, group_off, None, a, pairs), down_b, expert_of)
    if residual is not None:
        return ops.moe_combine(y, pair_of, w, b, k, out=residual, accumulate=True)
    return ops.moe_combine(y, pair_of, w, b, k)


def experts_forward_grouped(layer, x, group_off, gather, pairs, ops=None):
    """gate/up/GLU/down for `pairs` permuted rows grouped by expert (`grouped_proj` x3)."""
    ops = _ops(ops)
    g = ops.gemm_grouped(layer.gate, group_off, gather, x, pairs)
    u = ops.gemm_grouped(layer.up, group_off, gather, x, pairs)
    a = ops.glu(g, u, layer.act)
    return ops.gemm_grouped(layer.down, group_off, None, a, pairs)


def run_device_routed_batch(layer, x, ops=None):
    """Prefill: x [batch, hidden].  Pairs are grouped by expert (tokens ascending
    inside a group), each projection is ONE grouped GEMM over all experts."""
    ops = _ops(ops)
    if hasattr(ops, "moe_layer") and x.shape[0] > 8:
        return ops.moe_layer(layer, x)
    batch = x.shape[0]
    ids, w = route(layer, x, ops)
    group_off, gather, pair_of = ops.moe_permute(ids, layer.n_experts)
    y = experts_forward_grouped(layer, x, group_off, gather, batch * layer.k, ops)
    return ops.moe_combine(y, pair_of, w, batch, layer.k)


def routed_batch_supported(batch):
    """`prefill::routed_batch_supported`: from this batch on the grouped GEMM path is taken."""
    return batch > 8
