"""A minimal resident decoder over the quantized matmuls: what frink-models'
CUDA glue drives through `frink_cuda::prefill::launch_stack`
(crates/frink-models/src/decoder/cuda_prefill.rs:89, crates/frink-cuda/src/prefill/
layer.rs:44 `run_layer_resident`), reduced to the dense Llama graph and the
Qwen3-MoE graph: RMSNorm -> q/k/v -> RoPE -> KV append -> causal GQA -> wo ->
residual -> RMSNorm -> SwiGLU FFN or routed experts -> residual; final norm,
output head, greedy argmax.  Everything stays on the device; the position is a
device word so one decode step can be captured in a CUDA graph and replayed.

With a process group, dense projections are tensor parallel (q/k/v/gate/up split
by rows = heads, wo/down split by columns, one all-reduce each) and routed
experts are expert parallel (`parallel.ExpertParallelLayer.decode`)."""
from dataclasses import dataclass, field
from typing import Any, List, Optional

import numpy as np
import torch

from . import parallel
from .prefill import RoutedLayer, run_device_routed, run_device_routed_batch, run_device_routed_oai, run_device_routed_rows


@dataclass
class DecoderConfig:
    n_layers: int
    hidden: int
    n_heads: int
    n_kv: int
    head_dim: int
    ffn: int
    vocab: int
    rope_theta: float = 500000.0
    eps: float = 1e-5
    neox: bool = False          # Llama: adjacent pairs; Qwen3: split halves
    qk_norm: bool = False       # Qwen3 per-head RMSNorm on q and k
    n_experts: int = 0          # > 0: routed FFN
    top_k: int = 0
    route_mode: int = 1
    oai: bool = False           # gpt-oss layers: biased projections, biased experts with the clamped SwiGLU, router bias
    sliding_window: int = 0     # gpt-oss: > 0 = windowed layers see only this many most recent keys
    swa_period: int = 0         # which layers are windowed: all (0), or layer i with i % period < period - 1 (gpt-oss: 2)

    def window_of(self, layer):
        if self.sliding_window <= 0:
            return 0
        return self.sliding_window if self.swa_period <= 0 or layer % self.swa_period < self.swa_period - 1 else 0


@dataclass
class LayerWeights:
    """GGUF bytes (numpy uint8) + kinds of one layer; norms as f32 numpy."""
    attn_norm: Any
    wq: Any
    wk: Any
    wv: Any
    wo: Any
    ffn_norm: Any
    gate: Any = None
    up: Any = None
    down: Any = None
    router: Any = None          # f32 [n_experts, hidden]
    q_norm: Any = None
    k_norm: Any = None
    sinks: Any = None           # gpt-oss attention sinks, f32 [n_heads]
    bq: Any = None              # gpt-oss biases: q / k / v / attention output rows, the router's, and [n_experts, rows] per expert projection
    bk: Any = None
    bv: Any = None
    bo: Any = None
    router_bias: Any = None
    gate_b: Any = None
    up_b: Any = None
    down_b: Any = None
    kinds: dict = field(default_factory=dict)   # name -> fk_kind


def bf16_as_f32(ops, raw, kind, rows, cols):
    """BF16 weights widened to an f32 matrix on the device, for a prompt's rows: this library has no BF16 GEMM, and a
    plain f32 GEMM is the math library's (cuBLAS through torch; TF32 off, so the products are the matvec's).  None for
    every other kind and off the GPU."""
    if kind != 30 or getattr(ops, "__name__", "") != "frink_b200.device":
        return None
    import numpy as np
    bits = torch.from_numpy(np.ascontiguousarray(raw, np.uint8).ravel().view(np.uint16).astype(np.int32)).cuda()
    return (bits << 16).view(torch.float32).view(rows, cols)


def prefill_gemm(ops, w, x, acts):
    """The GEMM of a prompt's rows.  acts = "q8_k": Q4_K weights take the GEMM on Q8_K activations (frink's CPU
    activation rule, about twice as fast here); every other kind, and acts = "q8_1", the q8_1 GEMM whose integers
    are the decode matvec's."""
    if acts == "q8_k" and w.kind == 12 and hasattr(ops, "gemm_q8k"):
        return ops.gemm_q8k(w, x)
    return ops.gemm(w, x)


class _Linear:
    """rows x cols projection, batch <= 8 through the GEMV, above through the GEMM."""

    def __init__(self, ops, raw, kind, rows, cols, acts="q8_1"):
        self.ops, self.acts = ops, acts
        self.w = ops.Weights(raw, kind, rows, cols)
        self.w32 = bf16_as_f32(ops, raw, kind, rows, cols)

    def __call__(self, x):
        if x.shape[0] <= 8:
            return self.ops.gemv(self.w, x)
        return x @ self.w32.T if self.w32 is not None else prefill_gemm(self.ops, self.w, x, self.acts)


class _Merged:
    """Projections that read the same input and share a block format, stacked by rows
    into one weight handle: one launch (and one activation quantization) instead of
    several, as the reference shares one quantized input between q/k/v and gate/up
    (crates/frink-cuda/src/dp4a_launch.rs:56-62).  Returns the outputs as column slices."""

    def __init__(self, ops, parts, kind, cols, interleave=False, acts="q8_1"):
        import numpy as np
        self.ops, self.splits, self.interleave, self.acts = ops, [r for _, r in parts], interleave, acts
        blobs = [np.ascontiguousarray(b, np.uint8).ravel() for b, _ in parts]
        if interleave:
            # two projections of equal height, row i of the first then row i of the second: a lane of the
            # matvec then holds a (gate, up) pair and can write the gated activation itself
            assert len(parts) == 2 and self.splits[0] == self.splits[1]
            rows = self.splits[0]
            raw = np.stack([blobs[0].reshape(rows, -1), blobs[1].reshape(rows, -1)], axis=1).reshape(-1)
        else:
            raw = np.concatenate(blobs)
        self.w = ops.Weights(raw, kind, sum(self.splits), cols)
        self.w32 = bf16_as_f32(ops, raw, kind, sum(self.splits), cols)

    def __call__(self, x):
        if x.shape[0] <= 8:
            y = self.ops.gemv(self.w, x)
        else:
            y = x @ self.w32.T if self.w32 is not None else prefill_gemm(self.ops, self.w, x, self.acts)
        if self.interleave:
            return [y[:, 0::2], y[:, 1::2]]
        outs, o = [], 0
        for r in self.splits:
            outs.append(y[:, o:o + r] if x.shape[0] == 1 else y[:, o:o + r].contiguous())
            o += r
        return outs


class Decoder:
    def __init__(self, cfg: DecoderConfig, layers: List[LayerWeights], tok_embd, tok_kind, out_norm, output=None, output_kind=None,
                 max_seq=1024, ops=None, group=None, device="cuda", dense_parallel=True, comm=None, prefill_acts="q8_1"):
        """dense_parallel=False: attention and dense projections are replicated on every rank
        (no collectives for them) and only the routed experts are sharded over the group --
        the plan for MoE models whose KV heads do not divide by the number of ranks.
        comm (`frink_b200.comm.Comm`): decode rows are summed across ranks by the peer-memory
        all-reduce; without it every sum is a `torch.distributed` all-reduce.
        prefill_acts: "q8_1" (default: prompt rows are quantized by the decode rule, one set of integers for
        prefill and decode) or "q8_k" (Q4_K projections of a prompt take the faster GEMM on frink's CPU
        activation rule; decode is unchanged)."""
        if ops is None:
            from . import device as ops
        self.cfg, self.ops, self.group, self.dev = cfg, ops, group, device
        self.comm = comm
        self.rank, self.world = parallel._world(group) if group is not None or torch.distributed.is_initialized() else (0, 1)
        T = self.world if dense_parallel else 1
        self.t_dense = T
        r_dense = self.rank if dense_parallel else 0     # replicated: every rank holds shard 0 of 1
        E = self.world          # ranks the routed experts are spread over
        if cfg.oai and T > 1:
            raise ValueError("the gpt-oss layer form has no tensor-parallel variant (its projection biases are not sharded): "
                             "run it with dense_parallel=False (attention replicated, experts spread over the ranks)")
        if cfg.n_heads % T or cfg.n_kv % T:
            raise ValueError(f"{cfg.n_heads}/{cfg.n_kv} heads do not split over {T} ranks")
        self.h_loc, self.kv_loc = cfg.n_heads // T, cfg.n_kv // T
        hd, H = cfg.head_dim, cfg.hidden
        f32 = lambda a: torch.as_tensor(a, dtype=torch.float32).to(device).contiguous()
        self.embd = ops.Weights(tok_embd, tok_kind, cfg.vocab, H)
        self.head = self.embd if output is None else ops.Weights(output, output_kind, cfg.vocab, H)
        self.out_norm = f32(out_norm)
        self.layers = []
        for L in layers:
            k = L.kinds
            d = {"attn_norm": f32(L.attn_norm), "ffn_norm": f32(L.ffn_norm)}
            # q/k/v (and gate/up) as row shards of this rank, stacked where the formats agree
            sh = lambda raw, kind, rows: parallel.shard_rows(raw, kind, rows, H, r_dense, T)
            qkv = [(sh(L.wq, k["wq"], cfg.n_heads * hd), k["wq"]), (sh(L.wk, k["wk"], cfg.n_kv * hd), k["wk"]),
                   (sh(L.wv, k["wv"], cfg.n_kv * hd), k["wv"])]
            if k["wq"] == k["wk"] == k["wv"]:
                d["qkv"] = _Merged(ops, [p for p, _ in qkv], k["wq"], H, acts=prefill_acts)
            elif k["wq"] == k["wk"]:
                d["qk"] = _Merged(ops, [qkv[0][0], qkv[1][0]], k["wq"], H, acts=prefill_acts)
                d["wv"] = _Linear(ops, qkv[2][0][0], k["wv"], qkv[2][0][1], H, acts=prefill_acts)
            else:
                for name, ((raw, rows), kind) in zip(("wq", "wk", "wv"), qkv):
                    d[name] = _Linear(ops, raw, kind, rows, H, acts=prefill_acts)
            if T == 1:
                d["wo"] = _Linear(ops, L.wo, k["wo"], H, cfg.n_heads * hd, acts=prefill_acts)
            else:
                d["wo"] = parallel.RowParallelLinear(ops, L.wo, k["wo"], H, cfg.n_heads * hd, group, input_is_sharded=True, comm=comm, prefill_acts=prefill_acts)
            if cfg.qk_norm:
                d["q_norm"], d["k_norm"] = f32(L.q_norm), f32(L.k_norm)
            # attention options of the layer: the window (0 = full) and this rank's heads' sinks
            d["window"] = cfg.window_of(len(self.layers))
            d["sinks"] = None if L.sinks is None else f32(np.asarray(L.sinks, np.float32)[r_dense * self.h_loc:(r_dense + 1) * self.h_loc])
            if cfg.oai:
                for name in ("bq", "bk", "bv", "bo"):
                    if getattr(L, name) is not None:
                        d[name] = f32(getattr(L, name))
                # the bias rows of the stacked projections, stacked the same way (the decode form adds them in the matvec)
                if "qkv" in d and all(n_ in d for n_ in ("bq", "bk", "bv")):
                    d["bqkv"] = torch.cat([d["bq"], d["bk"], d["bv"]])
                elif "qk" in d and "bq" in d and "bk" in d:
                    d["bqk"] = torch.cat([d["bq"], d["bk"]])
            if cfg.n_experts and cfg.oai and E > 1:
                d["ep"] = parallel.ExpertParallelLayer(ops, f32(L.router), L.gate, L.up, L.down, k["experts"], cfg.n_experts, H, cfg.ffn,
                                                       cfg.top_k, mode=cfg.route_mode, act=1, group=group, comm=comm,
                                                       router_bias=None if L.router_bias is None else f32(L.router_bias),
                                                       biases=(f32(L.gate_b), f32(L.up_b), f32(L.down_b)))
            elif cfg.n_experts and cfg.oai:
                mk = lambda raw, r, c: ops.Weights(raw, k["experts"], r, c, n_mats=cfg.n_experts)
                d["moe"] = RoutedLayer(f32(L.router), mk(L.gate, cfg.ffn, H), mk(L.up, cfg.ffn, H), mk(L.down, H, cfg.ffn), k=cfg.top_k,
                                       mode=cfg.route_mode, act=1, router_bias=None if L.router_bias is None else f32(L.router_bias))
                d["moe_b"] = (f32(L.gate_b), f32(L.up_b), f32(L.down_b))
            elif cfg.n_experts:
                router = f32(L.router)
                if E == 1:
                    mk = lambda raw, r, c: ops.Weights(raw, k["experts"], r, c, n_mats=cfg.n_experts)
                    d["moe"] = RoutedLayer(router, mk(L.gate, cfg.ffn, H), mk(L.up, cfg.ffn, H), mk(L.down, H, cfg.ffn), k=cfg.top_k,
                                           mode=cfg.route_mode)
                else:
                    d["ep"] = parallel.ExpertParallelLayer(ops, router, L.gate, L.up, L.down, k["experts"], cfg.n_experts, H, cfg.ffn,
                                                           cfg.top_k, mode=cfg.route_mode, group=group, comm=comm)
            else:
                gu = [parallel.shard_rows(L.gate, k["gate"], cfg.ffn, H, r_dense, T), parallel.shard_rows(L.up, k["up"], cfg.ffn, H, r_dense, T)]
                if k["gate"] == k["up"]:
                    d["gate_up"] = _Merged(ops, gu, k["gate"], H, interleave=True, acts=prefill_acts)
                else:
                    d["gate"] = _Linear(ops, gu[0][0], k["gate"], gu[0][1], H, acts=prefill_acts)
                    d["up"] = _Linear(ops, gu[1][0], k["up"], gu[1][1], H, acts=prefill_acts)
                if T == 1:
                    d["down"] = _Linear(ops, L.down, k["down"], H, cfg.ffn, acts=prefill_acts)
                else:
                    d["down"] = parallel.RowParallelLinear(ops, L.down, k["down"], H, cfg.ffn, group, input_is_sharded=True, comm=comm, prefill_acts=prefill_acts)
            d["k"] = torch.zeros((max_seq, self.kv_loc * hd), dtype=torch.float32, device=device)
            d["v"] = torch.zeros((max_seq, self.kv_loc * hd), dtype=torch.float32, device=device)
            self.layers.append(d)
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.max_seq = max_seq
        self._pos_host = 0          # the device position's host mirror: what the cache capacity is checked against
        self._graph = None

    def reset(self):
        self.pos.zero_()
        self._pos_host = 0

    def _claim(self, n):
        """Refuse, before anything is launched, rows that would run past the KV caches."""
        if self._pos_host + n > self.max_seq:
            raise ValueError(f"{n} more rows at position {self._pos_host} do not fit KV caches of {self.max_seq} rows")
        self._pos_host += n

    # ---- one forward over n rows (token ids on the device); returns logits of the last row
    def forward(self, ids):
        ops, cfg = self.ops, self.cfg
        hd = cfg.head_dim
        n = ids.numel()
        self._claim(n)
        if n <= 8 and hasattr(ops, "gemv_fused") and (self.t_dense == 1 or self.comm is not None):
            return self._forward_fused(ids)
        x = ops.get_rows(self.embd, ids)                    # residual stream [n, hidden]
        pending = None                                      # a block output not yet added to x
        for L in self.layers:
            h = ops.rmsnorm(x, L["attn_norm"], cfg.eps, residual=pending)
            if "qkv" in L:
                q, k, v = L["qkv"](h)
            elif "qk" in L:
                (q, k), v = L["qk"](h), L["wv"](h)
            else:
                q, k, v = L["wq"](h), L["wk"](h), L["wv"](h)
            if "bq" in L:
                q, k, v = (ops.add_bias_(t_.contiguous(), L[b_]) for t_, b_ in ((q, "bq"), (k, "bk"), (v, "bv")))
            if cfg.qk_norm:
                q = ops.rmsnorm(q.view(-1, hd), L["q_norm"], cfg.eps).view(n, -1)
                k = ops.rmsnorm(k.view(-1, hd), L["k_norm"], cfg.eps).view(n, -1)
            if hasattr(ops, "rope_kv"):
                ops.rope_kv(q, k, v, self.h_loc, self.kv_loc, hd, self.pos, cfg.rope_theta, cfg.neox, L["k"], L["v"])
            else:
                ops.rope(q, self.h_loc, hd, self.pos, cfg.rope_theta, cfg.neox)
                ops.rope(k, self.kv_loc, hd, self.pos, cfg.rope_theta, cfg.neox)
                ops.kv_append(L["k"], k, self.pos)
                ops.kv_append(L["v"], v, self.pos)
            a = ops.attention(q, L["k"], L["v"], self.h_loc, self.kv_loc, hd, self.pos, window=L["window"], sinks=L["sinks"])
            o = L["wo"](a)
            if "bo" in L:
                ops.add_bias_(o, L["bo"])
            h2 = ops.rmsnorm(x, L["ffn_norm"], cfg.eps, residual=o)
            if "moe_b" in L:
                pending = run_device_routed_oai(L["moe"], L["moe_b"], h2, ops)
            elif "moe" in L:
                pending = run_device_routed(L["moe"], h2, ops) if n <= 8 else run_device_routed_batch(L["moe"], h2, ops)
            elif "ep" in L:
                pending = torch.stack([L["ep"].decode(h2[t]) for t in range(n)]) if n <= 8 else self._ep_prefill(L["ep"], h2)
            else:
                g_, u_ = L["gate_up"](h2) if "gate_up" in L else (L["gate"](h2), L["up"](h2))
                pending = L["down"](ops.glu(g_.contiguous(), u_.contiguous(), 0))
        last = x[n - 1:n].contiguous()
        hn = ops.rmsnorm(last, self.out_norm, cfg.eps, residual=pending[n - 1:n].contiguous())
        logits = ops.gemv(self.head, hn)
        ops.add_int_(self.pos, n)
        return logits

    # ---- batched decode: several independent sequences, one token each per step
    def alloc_seqs(self, n_seqs):
        """KV caches and positions for n_seqs (<= 8) independent sequences, decoded together by `forward_seqs`."""
        if not 1 <= n_seqs <= 8:
            raise ValueError("a decode batch holds 1 to 8 sequences")
        for L in self.layers:
            L["ks"] = torch.zeros((n_seqs,) + tuple(L["k"].shape), dtype=torch.float32, device=L["k"].device)
            L["vs"] = torch.zeros_like(L["ks"])
        self.seq_pos = torch.zeros(n_seqs, dtype=torch.int32, device=self.pos.device)
        self._seq_pos_host = [0] * n_seqs

    def prefill_seq(self, s, prompt_ids):
        """Sequence s's prompt through the ordinary forward, on that sequence's caches -> its first generated token."""
        saved = [(L["k"], L["v"]) for L in self.layers]
        pos0, host0 = self.pos.clone(), self._pos_host
        try:
            for L in self.layers:
                L["k"], L["v"] = L["ks"][s], L["vs"][s]
            self.reset()
            tok = self.ops.argmax(self.forward(prompt_ids))
            self.seq_pos[s:s + 1].copy_(self.pos)
            self._seq_pos_host[s] = self._pos_host
        finally:
            for L, (k_, v_) in zip(self.layers, saved):
                L["k"], L["v"] = k_, v_
            self.pos.copy_(pos0)
            self._pos_host = host0
        return tok

    def forward_seqs(self, toks):
        """toks [n_seqs] (device int32), sequence r's newest token -> logits [n_seqs, vocab]; every position advances."""
        n = toks.numel()
        if n != len(self._seq_pos_host):
            raise ValueError(f"{n} tokens for {len(self._seq_pos_host)} sequences")
        if max(self._seq_pos_host) + 1 > self.max_seq:
            raise ValueError(f"a sequence at position {max(self._seq_pos_host)} has filled its KV cache of {self.max_seq} rows")
        self._seq_pos_host = [p + 1 for p in self._seq_pos_host]
        return self._forward_fused(toks, seqs=True)

    def capture_decode_seqs(self, toks):
        """`forward_seqs` + argmax captured in a CUDA graph (reads `toks`, returns the graph and the next tokens)."""
        pos0, host0 = self.seq_pos.clone(), list(self._seq_pos_host)
        if max(host0) + 2 > self.max_seq:
            raise ValueError("capturing needs two free rows in every KV cache (the warm-up steps write there)")
        for _ in range(2):
            self.ops.argmax(self.forward_seqs(toks))
        self.seq_pos.copy_(pos0)
        self._seq_pos_host = list(host0)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self.ops.argmax(self.forward_seqs(toks))
        self.seq_pos.copy_(pos0)
        self._seq_pos_host = list(host0)
        self._graph_seqs = g
        return g, out

    def replay_seqs(self):
        if max(self._seq_pos_host) + 1 > self.max_seq:
            raise ValueError(f"a sequence has filled its KV cache of {self.max_seq} rows")
        self._seq_pos_host = [p + 1 for p in self._seq_pos_host]
        self._graph_seqs.replay()

    def _forward_fused(self, ids, seqs=False):
        """The decode form (at most 8 rows): each RMSNorm rides in the prologue of the matvec that
        reads it, SiLU(gate) * up in the prologue of the down projection, and wo / down add
        straight into the residual stream; q, k, v stay column slices of the merged projection's
        output.  Six launches per dense layer.  Tensor-parallel (with a `Comm`): the same six
        launches on this rank's heads and FFN columns; wo and down are row-split and their
        matvec's epilogue sums the partial rows over the ranks through peer memory, so the
        residual stream stays replicated (and bit-identical) on every rank."""
        ops, cfg = self.ops, self.cfg

        def into_residual(lin, inp, is_padded=False, **kw):
            if kw.get("bias") is None:
                kw.pop("bias", None)
            if isinstance(lin, parallel.RowParallelLinear):
                ops.gemv_fused(lin.w, inp if is_padded else lin.padded(inp), out=x, accumulate=True, allreduce=(lin.comm, lin.ch), **kw)
            else:
                ops.gemv_fused(lin.w, inp, out=x, accumulate=True, **kw)

        hd, n = cfg.head_dim, ids.numel()
        hq, kvw = self.h_loc * hd, self.kv_loc * hd
        x = ops.get_rows(self.embd, ids)
        for L in self.layers:
            def normed(name, bias=None):
                # the attention norm rides in the prologue of every projection that reads it, a gpt-oss bias row in its epilogue
                kw = {} if L.get(bias) is None else {"bias": L[bias]}
                return ops.gemv_fused(L[name].w, x, norm_weight=L["attn_norm"], eps=cfg.eps, **kw)
            if "qkv" in L:
                qkv = normed("qkv", "bqkv")
                q, k, v = qkv[:, :hq], qkv[:, hq:hq + kvw], qkv[:, hq + kvw:]
            elif "qk" in L:
                # v in another block format (the usual K-quant mix): two matvecs, the norm folded into both
                qk = normed("qk", "bqk")
                q, k = qk[:, :hq], qk[:, hq:hq + kvw]
                v = normed("wv", "bv")
            else:
                q, k, v = normed("wq", "bq"), normed("wk", "bk"), normed("wv", "bv")
            window = getattr(L["wo"], "window", None)
            if seqs:
                a = ops.attention_rope_kv_seqs(q, k, v, L["ks"], L["vs"], self.h_loc, self.kv_loc, hd, self.seq_pos, cfg.rope_theta, cfg.neox,
                                               q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=cfg.eps, window=L["window"], sinks=L["sinks"])
            elif n == 1 and hasattr(ops, "attention_rope_kv") and window is not None:
                # this rank's heads are a K range cut inside the blocks of wo: attention writes straight into the window
                # of the zero-padded row the local product reads
                if not hasattr(L["wo"], "row"):
                    L["wo"].row = torch.zeros((1, L["wo"].cols_local), dtype=torch.float32, device=x.device)
                ops.attention_rope_kv(q, k, v, L["k"], L["v"], self.h_loc, self.kv_loc, hd, self.pos, cfg.rope_theta, cfg.neox,
                                      q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=cfg.eps,
                                      out=L["wo"].row[:, window[0]:window[0] + window[1]], window=L["window"], sinks=L["sinks"])
                a = None
            elif n == 1 and hasattr(ops, "attention_rope_kv"):
                a = ops.attention_rope_kv(q, k, v, L["k"], L["v"], self.h_loc, self.kv_loc, hd, self.pos, cfg.rope_theta, cfg.neox,
                                          q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=cfg.eps, window=L["window"], sinks=L["sinks"])
            else:
                if n > 1 and k.stride(0) != v.stride(0):
                    k, v = k.contiguous(), v.contiguous()          # the cache append wants one row stride for both
                ops.rope_kv(q, k, v, self.h_loc, self.kv_loc, hd, self.pos, cfg.rope_theta, cfg.neox, L["k"], L["v"],
                            q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=cfg.eps)
                a = ops.attention(q, L["k"], L["v"], self.h_loc, self.kv_loc, hd, self.pos, window=L["window"], sinks=L["sinks"])
            if a is None:
                into_residual(L["wo"], L["wo"].row, is_padded=True)
            else:
                into_residual(L["wo"], a, bias=L.get("bo"))
            if ("moe" in L or "moe_b" in L) and hasattr(ops, "moe_layer"):
                # the whole routed layer on the residual stream: the norm rides in the router and in the gate / up launch
                ops.moe_layer(L["moe"], x, out=x, accumulate=True, biases=L.get("moe_b"), norm=(L["ffn_norm"], cfg.eps))
            elif "moe_b" in L:
                h2 = ops.rmsnorm(x, L["ffn_norm"], cfg.eps)
                run_device_routed_oai(L["moe"], L["moe_b"], h2, ops, residual=x)
            elif "moe" in L:
                h2 = ops.rmsnorm(x, L["ffn_norm"], cfg.eps)
                if n > 1 and hasattr(ops, "gemv_multi_glu"):
                    run_device_routed_rows(L["moe"], h2, ops, residual=x)      # all rows' (row, expert) pairs as slots of one launch
                else:
                    run_device_routed(L["moe"], h2, ops, residual=x)
            elif "ep" in L:
                # experts spread over the ranks, everything else replicated: the one collective of the layer
                h2 = ops.rmsnorm(x, L["ffn_norm"], cfg.eps)
                if n > 1:
                    ops.add_(x, L["ep"].decode_rows(h2))
                else:
                    ops.add_(x[0], L["ep"].decode(h2[0]))
            elif "gate_up" in L:
                act = ops.gemv_fused(L["gate_up"].w, x, norm_weight=L["ffn_norm"], eps=cfg.eps, pair_glu=1)
                into_residual(L["down"], act)
            else:
                h2 = ops.rmsnorm(x, L["ffn_norm"], cfg.eps)
                into_residual(L["down"], L["gate"](h2), glu_up=L["up"](h2))
        if seqs:
            logits = ops.gemv_fused(self.head, x, norm_weight=self.out_norm, eps=cfg.eps)
            self.seq_pos.add_(1)
            return logits
        logits = ops.gemv_fused(self.head, x[n - 1:n], norm_weight=self.out_norm, eps=cfg.eps)
        ops.add_int_(self.pos, n)
        return logits

    def _ep_prefill(self, ep, h2):
        """Activations are replicated, so every rank holds all rows: each routes them all, serves the pairs of
        its own experts and the partial sums are all-reduced (`ExpertParallelLayer.prefill_replicated`)."""
        return ep.prefill_replicated(h2)

    def prefill(self, ids):
        """Prompt of S token ids -> the first generated token (device int32 [1])."""
        return self.ops.argmax(self.forward(ids))

    def decode_step(self, tok):
        return self.ops.argmax(self.forward(tok))

    def capture_decode(self, tok):
        """Capture one decode step (reads `tok`, writes the returned tensor, advances
        the position word) into a CUDA graph; `replay()` runs it again."""
        pos0, host0 = self.pos.clone(), self._pos_host
        if host0 + 2 > self.max_seq:
            raise ValueError(f"capturing at position {host0} needs two free rows in KV caches of {self.max_seq} rows (the warm-up steps write there)")
        for _ in range(2):                      # warm up outside the capture, then put the position back
            self.decode_step(tok)
        self.pos.copy_(pos0)
        self._pos_host = host0
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self.decode_step(tok)
        self.pos.copy_(pos0)
        self._pos_host = host0
        self._graph, self._gout = g, out
        return g, out

    def replay(self):
        """One more step of the captured graph (the position advances on the device and in its host mirror)."""
        self._claim(1)
        self._graph.replay()

    def generate(self, prompt_ids, n_new, use_graph=False):
        """Greedy: returns the n_new generated token ids (list of int)."""
        tok = self.prefill(prompt_ids)
        outs = [tok.clone()]
        if use_graph and n_new > 1:
            cur = tok.clone()
            g, out = self.capture_decode(cur)
            for _ in range(n_new - 1):
                self.replay()
                cur.copy_(out)
                outs.append(out.clone())
        else:
            for _ in range(n_new - 1):
                tok = self.decode_step(tok)
                outs.append(tok.clone())
        return [int(t.item()) for t in outs]
