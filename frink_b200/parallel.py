"""Multi-GPU sharding of the path: tensor parallel for dense projections,
expert parallel for routed layers, one process per GPU over `torch.distributed`
(NCCL on the GPUs, gloo in the CPU tests).

The reference is single-device (crates/frink-cuda/src/gpu.rs:219; "tensor,
pipeline and multi-node parallelism" are under "Not now",
docs/plans/north-star.md:170-174), so nothing here mirrors reference code; it
shards the reference's tensors so that every rank's local work is the
single-GPU path unchanged.

* Column split (`shard_rows`): a rank holds whole quantized rows -- wq/wk/wv,
  gate/up.  No communication; the activation is replicated.
* Row split (`shard_cols`): a rank holds a K range of every row, cut on block
  boundaries (a q8_1 run never straddles a cut, so every per-run integer is the
  single-GPU integer) -- wo/down.  Partial outputs are all-reduced (sum, f32).
* Experts: rank r owns experts [r E/P, (r+1) E/P).  Decode (activation
  replicated): each rank runs the chosen experts it owns and the weighted
  partial sums are all-reduced.  Prefill with tokens sharded over ranks: rows
  travel to their experts' owners and back with two all-to-alls, and the source
  combines them in routing order, which reproduces the single-GPU result
  bit for bit.

`ops` is the compute backend (`frink_b200.device` on GPUs)."""
import numpy as np
import torch
import torch.distributed as dist

BLOCK = {8: (34, 32), 12: (144, 256), 13: (176, 256), 14: (210, 256), 39: (17, 32), 30: (2, 1)}   # kind -> (bytes, elems)


def shard_rows(raw, kind, rows, cols, rank, world):
    """GGUF bytes of rows [rank rows/world, (rank+1) rows/world) -> (bytes, local rows)."""
    if rows % world:
        raise ValueError(f"{rows} rows do not split over {world} ranks")
    bb, be = BLOCK[kind]
    rb = cols // be * bb
    lo = rank * (rows // world)
    raw = np.ascontiguousarray(raw, np.uint8).ravel()
    return raw[lo * rb:(lo + rows // world) * rb], rows // world


def shard_cols(raw, kind, rows, cols, rank, world):
    """GGUF bytes of the K range [rank cols/world, (rank+1) cols/world) of every row,
    cut on block boundaries -> (bytes, local cols).  Refused when a cut would fall
    inside a block (e.g. 3072 columns of a 256-wide format over 8 ranks)."""
    bb, be = BLOCK[kind]
    nblk = cols // be
    if nblk % world:
        raise ValueError(f"{nblk} blocks of {be} per row do not split over {world} ranks")
    per = nblk // world
    m = np.ascontiguousarray(raw, np.uint8).reshape(rows, nblk, bb)
    return np.ascontiguousarray(m[:, rank * per:(rank + 1) * per]).ravel(), per * be


def mask_outside(raw, kind, rows, cols, lo, hi):
    """The GGUF bytes with everything outside columns [lo, hi) made to contribute exactly zero, without
    touching a quant: Q4_K sub-blocks of 32 get scale 0 and min 0, Q6_K groups of 16 get scale 0.  lo and hi
    are multiples of 32 (Q4_K) / 16 (Q6_K).  The integers of the columns inside are untouched, so a product
    with the masked matrix is the single-GPU product restricted to the window."""
    bb, be = BLOCK[kind]
    m = np.ascontiguousarray(raw, np.uint8).reshape(rows, cols // be, bb).copy()
    if kind == 12:
        if lo % 32 or hi % 32:
            raise ValueError("a Q4_K window is cut in units of 32 columns")
        sc = m[:, :, 4:16]                      # 8 six-bit scales and 8 six-bit mins in 12 bytes
        for j in range(cols // 32):
            if lo <= j * 32 < hi:
                continue
            b, k = divmod(j, 8)
            if k < 4:                           # low six bits of bytes k (scale) and k + 4 (min)
                sc[:, b, k] &= 0xC0
                sc[:, b, k + 4] &= 0xC0
            else:                               # byte k + 4 (low nibbles) and the top two bits of bytes k - 4, k
                sc[:, b, k + 4] = 0
                sc[:, b, k - 4] &= 0x3F
                sc[:, b, k] &= 0x3F
    elif kind == 14:
        if lo % 16 or hi % 16:
            raise ValueError("a Q6_K window is cut in units of 16 columns")
        sc = m[:, :, 192:208]                   # 16 int8 scales, one per 16 columns in order
        for j in range(cols // 16):
            if not lo <= j * 16 < hi:
                sc[:, j // 16, j % 16] = 0
    else:
        raise ValueError("32-wide formats are cut on block boundaries; no mask is needed")
    return m.ravel()


def shard_cols_window(raw, kind, rows, cols, rank, world):
    """The K range [rank cols/world, (rank+1) cols/world) of every row when it does not fall on the format's
    block boundaries (3072 columns of a 256-wide format over 8 ranks: 384 columns a rank): the rank holds the
    whole blocks that cover its range, with the columns outside masked to contribute zero
    -> (bytes, local cols, offset of the range inside them, its width).  The input of the local product is
    the rank's activations at [offset, offset + width) of a row of local cols, anything finite elsewhere."""
    bb, be = BLOCK[kind]
    if cols % world or (cols // world) % 32:
        raise ValueError(f"{cols} columns do not split over {world} ranks in units of 32")
    w = cols // world
    lo, hi = rank * w, (rank + 1) * w
    b0, b1 = lo // be, (hi + be - 1) // be
    nb = max((((r + 1) * w + be - 1) // be) - (r * w) // be for r in range(world))   # the same width on every rank
    if b0 + nb > cols // be:
        b0 = cols // be - nb
    masked = mask_outside(raw, kind, rows, cols, lo, hi).reshape(rows, cols // be, bb)
    return np.ascontiguousarray(masked[:, b0:b0 + nb]).ravel(), nb * be, lo - b0 * be, w


def _world(group=None):
    if not dist.is_available() or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


class ColumnParallelLinear:
    """y_local = W[rows of this rank] x; `gather=True` all-gathers the row shards."""

    def __init__(self, ops, raw, kind, rows, cols, group=None, gather=False):
        self.ops, self.group, self.gather = ops, group, gather
        self.rank, self.world = _world(group)
        local, self.rows_local = shard_rows(raw, kind, rows, cols, self.rank, self.world)
        self.rows, self.cols = rows, cols
        self.w = ops.Weights(local, kind, self.rows_local, cols)

    def __call__(self, x):
        x2 = x if x.dim() == 2 else x[None]
        y = self.ops.gemv(self.w, x2) if x2.shape[0] <= 8 else self.ops.gemm(self.w, x2)
        if self.gather and self.world > 1:
            parts = [torch.empty_like(y) for _ in range(self.world)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=1)
        return y if x.dim() == 2 else y[0]


class RowParallelLinear:
    """y = sum over ranks of W[:, K range of the rank] x[K range]: one all-reduce."""

    def __init__(self, ops, raw, kind, rows, cols, group=None, input_is_sharded=False, comm=None, prefill_acts="q8_1"):
        """comm (`frink_b200.comm.Comm`): decode rows (at most 8) are summed by the peer-memory all-reduce
        instead of the library collective, whose fixed cost is several matvecs at these sizes."""
        self.ops, self.group, self.input_is_sharded, self.prefill_acts = ops, group, input_is_sharded, prefill_acts
        self.rank, self.world = _world(group)
        self.comm = comm if comm is not None and self.world > 1 else None
        self.ch = self.comm.channel(8 * rows) if self.comm else None
        bb, be = BLOCK[kind]
        self.window = None           # (offset, width) when the rank's K range is cut inside blocks
        if (cols // be) % self.world:
            local, self.cols_local, off, width = shard_cols_window(raw, kind, rows, cols, self.rank, self.world)
            self.window = (off, width)
        else:
            local, self.cols_local = shard_cols(raw, kind, rows, cols, self.rank, self.world)
        self.rows, self.cols = rows, cols
        self.w = ops.Weights(local, kind, rows, self.cols_local)

    def padded(self, x2):
        """x2 [n, width] (this rank's K range) as the [n, local cols] input of the local product."""
        if self.window is None:
            return x2
        off, width = self.window
        p = torch.zeros((x2.shape[0], self.cols_local), dtype=x2.dtype, device=x2.device)
        p[:, off:off + width] = x2
        return p

    def __call__(self, x):
        x2 = x if x.dim() == 2 else x[None]
        if not self.input_is_sharded:
            w_ = self.cols // self.world
            x2 = x2[:, self.rank * w_:(self.rank + 1) * w_].contiguous()
        x2 = self.padded(x2)
        if x2.shape[0] <= 8:
            y = self.ops.gemv(self.w, x2)
        elif self.prefill_acts == "q8_k" and self.w.kind == 12 and hasattr(self.ops, "gemm_q8k"):
            y = self.ops.gemm_q8k(self.w, x2)       # a K range cut inside blocks is masked by zeroed scales: exact here too
        else:
            y = self.ops.gemm(self.w, x2)
        if self.world > 1:
            if self.comm is not None and x2.shape[0] <= 8:
                self.comm.all_reduce(self.ch, y)
            else:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y if x.dim() == 2 else y[0]


class TensorParallelFFN:
    """SwiGLU FFN: gate/up column-split, down row-split, one all-reduce per call
    (the dense form of `gpu::launch_dense_ffn_swiglu`, sharded)."""

    def __init__(self, ops, gate_raw, up_raw, down_raw, kind_gu, kind_down, hidden, ffn, group=None):
        self.ops = ops
        self.gate = ColumnParallelLinear(ops, gate_raw, kind_gu, ffn, hidden, group)
        self.up = ColumnParallelLinear(ops, up_raw, kind_gu, ffn, hidden, group)
        self.down = RowParallelLinear(ops, down_raw, kind_down, hidden, ffn, group, input_is_sharded=True)

    def __call__(self, x):
        a = self.ops.glu(self.gate(x), self.up(x), 0)
        return self.down(a)


class ExpertParallelLayer:
    """A routed layer whose experts are split over the ranks of `group`."""

    def __init__(self, ops, router, gate_raw, up_raw, down_raw, kind, n_experts, hidden, ffn, k, mode=1, act=0, group=None, comm=None,
                 router_bias=None, biases=None):
        """router_bias [n_experts] and biases = (gate_b, up_b, down_b), each [n_experts, rows] (tensors on the ops' device):
        gpt-oss's form (`run_expert_oai`, crates/frink-moe/src/lib.rs:1039-1060) -- the router and its bias are replicated,
        every rank keeps the bias rows of its own experts."""
        from .prefill import RoutedLayer
        self.ops, self.group = ops, group
        self.rank, self.world = _world(group)
        self.comm = comm if comm is not None and self.world > 1 else None
        self.ch = self.comm.channel(8 * hidden) if self.comm else None
        if n_experts % self.world:
            raise ValueError(f"{n_experts} experts do not split over {self.world} ranks")
        self.n_experts, self.n_local = n_experts, n_experts // self.world
        self.e0 = self.rank * self.n_local
        self.hidden, self.ffn, self.k = hidden, ffn, k
        bb, be = BLOCK[kind]

        def local(raw, rows, cols):
            per = rows * (cols // be) * bb
            raw = np.ascontiguousarray(raw, np.uint8).ravel()
            return ops.Weights(raw[self.e0 * per:(self.e0 + self.n_local) * per], kind, rows, cols, n_mats=self.n_local)

        self.layer = RoutedLayer(router, local(gate_raw, ffn, hidden), local(up_raw, ffn, hidden), local(down_raw, hidden, ffn),
                                 k=k, mode=mode, act=act, n_experts=n_experts, router_bias=router_bias)
        # this rank's bias rows, and one row of zeros behind them: the group "some other rank's expert" of the prefill
        # permutation (and nothing else) indexes it
        self.biases = None
        if biases is not None:
            self.biases = tuple(torch.cat([b[self.e0:self.e0 + self.n_local], torch.zeros_like(b[:1])]).contiguous() for b in biases)

    def _bias(self, t, which, ids):
        """t [slots, rows] += this rank's bias row of every slot's (local) expert; nothing without biases."""
        if self.biases is not None:
            self.ops.add_bias_(t, self.biases[which], ids)
        return t

    # ---- decode: activation replicated, partial combine, one all-reduce
    def decode(self, x):
        from .prefill import route
        ops, L, k = self.ops, self.layer, self.k
        ids, w = route(L, x, ops)                       # replicated: every rank routes the same way
        if hasattr(ops, "moe_local_slots"):
            # all on the device: the chosen experts this rank owns move to the front, the
            # indexed matvecs skip the other slots, whose zeroed outputs carry weight 0
            lid, lw, n = ops.moe_local_slots(ids, w, self.e0, self.n_local)
            g = torch.zeros((k, self.ffn), dtype=torch.float32, device=x.device)
            u = torch.zeros_like(g)
            y = torch.zeros((k, self.hidden), dtype=torch.float32, device=x.device)
            # (slots past the count hold zeros plus expert 0's bias row: finite, and weighted by 0)
            self._bias(ops.gemv_multi_active(L.gate, lid, x, n, g), 0, lid)
            self._bias(ops.gemv_multi_active(L.up, lid, x, n, u), 1, lid)
            self._bias(ops.gemv_multi_active(L.down, lid, ops.glu(g, u, L.act), n, y), 2, lid)
            out = ops.moe_combine(y, None, lw[None], 1, k)[0]
        else:
            ids1, w1 = ids.reshape(-1), w.reshape(-1)
            mine = (ids1 >= self.e0) & (ids1 < self.e0 + self.n_local)
            out = torch.zeros(self.hidden, dtype=torch.float32, device=x.device)
            n = int(mine.sum().item())
            if n:
                lid = (ids1[mine] - self.e0).to(torch.int32).contiguous()
                g = self._bias(ops.gemv_multi(L.gate, lid, x), 0, lid)
                u = self._bias(ops.gemv_multi(L.up, lid, x), 1, lid)
                y = self._bias(ops.gemv_multi(L.down, lid, ops.glu(g, u, L.act)), 2, lid)
                out = ops.moe_combine(y, None, w1[mine].contiguous()[None], 1, n)[0]
        if self.world > 1:
            if self.comm is not None:
                self.comm.all_reduce(self.ch, out)
            else:
                dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out

    # ---- prefill over replicated activations: no dispatch at all.  Every rank holds every row (the decoder's
    # activations are replicated under tensor parallelism), routes all of them the same way, runs the pairs whose
    # expert it owns, and the weighted partial sums meet in ONE all-reduce.  No counts travel, nothing syncs
    # with the host, and every rank makes the same collective calls whatever the row count.
    def prefill_replicated(self, x):
        from .prefill import route
        ops, L, k = self.ops, self.layer, self.k
        b = x.shape[0]
        ids, w = route(L, x, ops)
        lids, lw = ops.moe_localize(ids, w, self.e0, self.n_local)
        # the pairs of other ranks' experts fall into a group past the last local expert, which no GEMM serves
        group_off, gather, pair_of = ops.moe_permute(lids, self.n_local + 1)
        pairs = b * k
        expert_of = None
        if self.biases is not None:
            # the (local) expert of every permuted row, from the group offsets; rows of other ranks' experts get the zero row
            expert_of = torch.searchsorted(group_off[1:].to(torch.int64), torch.arange(pairs, device=group_off.device), right=True)
            expert_of = expert_of.clamp_(max=self.n_local).to(torch.int32)
        g = self._bias(ops.gemm_grouped(L.gate, group_off, gather, x, pairs), 0, expert_of)
        u = self._bias(ops.gemm_grouped(L.up, group_off, gather, x, pairs), 1, expert_of)
        a = ops.glu(g, u, L.act)
        y = torch.zeros((pairs, self.hidden), dtype=torch.float32, device=x.device)   # rows nobody writes carry weight 0: keep them finite
        y = self._bias(ops.gemm_grouped(L.down, group_off, None, a, pairs, out=y), 2, expert_of)
        out = ops.moe_combine(y, pair_of, lw, b, k)
        if self.world > 1:
            if self.comm is not None and b <= 8:
                self.comm.all_reduce(self.ch, out)
            else:
                dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out

    def decode_rows(self, x):
        """A decode batch of independent rows x [b <= 8, hidden] (replicated on every rank): the (row, expert) pairs this
        rank's experts serve become the slots of one indexed launch per projection -- packed to the front on the device,
        the launches skip the rest -- and one all-reduce sums the weighted partial rows over the ranks."""
        from .prefill import route
        ops, L, k = self.ops, self.layer, self.k
        b = x.shape[0]
        if not hasattr(ops, "moe_local_pairs"):
            return self.prefill_replicated(x)
        ids, w = route(L, x, ops)
        lid, src, pair_of, lw, n = ops.moe_local_pairs(ids, w, self.e0, self.n_local)
        xg = x.index_select(0, src)                      # slot p reads the row its pair came from
        pairs = b * k
        if getattr(self, "_rows_buf", None) is None or self._rows_buf[0].shape[0] != pairs:
            # slots past the count are skipped by the launches: what they hold must stay finite (it is weighted by 0)
            self._rows_buf = (torch.zeros((pairs, self.ffn), dtype=torch.float32, device=x.device),
                              torch.zeros((pairs, self.ffn), dtype=torch.float32, device=x.device),
                              torch.zeros((pairs, self.hidden), dtype=torch.float32, device=x.device))
        g, u, y = self._rows_buf
        self._bias(ops.gemv_multi_active(L.gate, lid, xg, n, g), 0, lid)
        self._bias(ops.gemv_multi_active(L.up, lid, xg, n, u), 1, lid)
        self._bias(ops.gemv_multi_glu(L.down, lid, g, u, L.act, out=y, n_active=n), 2, lid)
        out = ops.moe_combine(y, pair_of, lw, b, k)
        if self.world > 1:
            if self.comm is not None:
                self.comm.all_reduce(self.ch, out)
            else:
                dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out

    # ---- prefill: tokens sharded over ranks, dispatch / combine all-to-all.  Every rank of the group must call
    # this, also with no rows of its own (it still serves its experts for the other ranks' rows).
    def prefill(self, x_local):
        from .prefill import experts_forward_grouped, route
        ops, L, k, P = self.ops, self.layer, self.k, self.world
        b = x_local.shape[0]
        if b:
            ids, w = route(L, x_local, ops)
        else:
            ids = torch.zeros((0, k), dtype=torch.int32, device=x_local.device)
            w = torch.zeros((0, k), dtype=torch.float32, device=x_local.device)
        ids1 = ids.reshape(-1).to(torch.int64)
        order = torch.argsort(ids1, stable=True)        # by expert, hence by owner rank; tokens ascending inside
        send_rows = x_local[(order // k)].contiguous()
        send_ids = ids1[order].to(torch.int32).contiguous()
        send_cnt = torch.bincount(ids1 // self.n_local, minlength=P).to(torch.int64)
        recv_cnt = torch.empty_like(send_cnt)
        if P > 1:
            dist.all_to_all_single(recv_cnt, send_cnt, group=self.group)
        else:
            recv_cnt.copy_(send_cnt)
        s_cnt, r_cnt = send_cnt.cpu().tolist(), recv_cnt.cpu().tolist()
        n_recv = int(sum(r_cnt))
        rows = torch.empty((n_recv, self.hidden), dtype=torch.float32, device=x_local.device)
        rids = torch.empty(n_recv, dtype=torch.int32, device=x_local.device)
        if P > 1:
            dist.all_to_all_single(rows, send_rows, r_cnt, s_cnt, group=self.group)
            dist.all_to_all_single(rids, send_ids, r_cnt, s_cnt, group=self.group)
        else:
            rows, rids = send_rows, send_ids
        y = torch.empty((n_recv, self.hidden), dtype=torch.float32, device=x_local.device)
        if n_recv:
            lid = (rids - self.e0).to(torch.int32).reshape(-1, 1).contiguous()
            group_off, gather, pair_of = ops.moe_permute(lid, self.n_local)
            yp = experts_forward_grouped(L, rows, group_off, gather, n_recv, ops)
            y = yp[pair_of.to(torch.int64)]            # back to arrival order
        back = torch.empty((b * k, self.hidden), dtype=torch.float32, device=x_local.device)
        if P > 1:
            dist.all_to_all_single(back, y.contiguous(), s_cnt, r_cnt, group=self.group)
        else:
            back = y
        if not b:
            return x_local.new_zeros((0, self.hidden))
        inv = torch.empty_like(order)
        inv[order] = torch.arange(b * k, device=order.device)
        return ops.moe_combine(back, inv.to(torch.int32), w, b, k)
