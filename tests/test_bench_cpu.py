"""bench.py's host-side tables: the bytes a decode token streams and the prompt FLOPs quoted for each synthetic model
shape must follow from the shape itself (block sizes of the kinds each tensor is stored in)."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("frink_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


# bytes per weight of the kinds the synthetic models store their tensors in
Q4_K, Q6_K, Q8_0, MXFP4, BF16, F32 = 144 / 256, 210 / 256, 34 / 32, 17 / 32, 2.0, 4.0


@pytest.mark.parametrize("name,attn,experts,head", [("qwen3moe", Q8_0, Q4_K, Q6_K), ("gptoss", BF16, MXFP4, BF16)])
def test_routed_model_roofline_figures_follow_from_the_shape(name, attn, experts, head):
    b = _bench()
    cfg = b.synth_model(name, 0)[0]
    H, hd = cfg.hidden, cfg.head_dim
    attn_w = (cfg.n_heads * hd + 2 * cfg.n_kv * hd) * H + H * cfg.n_heads * hd
    expert_w = cfg.top_k * 3 * cfg.ffn * H                      # the chosen experts' gate, up and down
    router_w = cfg.n_experts * H
    per_layer = attn_w * attn + expert_w * experts + router_w * F32
    want_bytes = cfg.n_layers * per_layer + cfg.vocab * H * head
    want_flops = 2 * 512 * cfg.n_layers * (attn_w + expert_w + router_w)
    got = b.MODEL_ROOFLINE[name]
    assert abs(got["bytes_per_token"] - want_bytes) <= 1e-6 * want_bytes
    assert abs(got["pp512_flops"] - want_flops) <= 5e-3 * want_flops
    assert got["one_gpu_only"]
