"""The allocation-free router entry point against the handle-based router.

Hosts that cannot call cudaMalloc (all free HBM already belongs to their expert pool, or they are inside
a decode loop that must not take cudaMalloc's device-wide synchronisation) route through
`shrike_encode_router_static`, whose logits scratch is a fixed array inside the library. It must give
the handle-based `shrike_encode_router` answer bit for bit (ids exact, weights exact: both run the same
kernels), on repeated calls that reuse the shared array, and refuse sizes beyond the array.

This file is collected last on purpose: a run that stops at the first failure has then run every other test.
"""
import numpy as np
import pytest
import torch

from gpu_harness import Layer, inputs, small_config, to_act_tensor
from shrike_b200 import capi
from shrike_b200.moe import ShrikeError, encode_router_static

pytestmark = pytest.mark.gpu


def route_both(layer: Layer, x: np.ndarray):
    cfg = layer.cfg
    x_dev = to_act_tensor(x, cfg.act_dtype, layer.device)
    ids, w, gate = layer.route(x_dev)
    ids2 = torch.full_like(ids, -1)
    w2 = torch.full_like(w, -1.0)
    gate2 = torch.full_like(gate, -1.0) if gate is not None else None
    encode_router_static(cfg, layer.router_ops, x_dev, ids2, w2, gate2)
    torch.cuda.synchronize()
    return (ids, w, gate), (ids2, w2, gate2)


@pytest.mark.parametrize("kw,T", [
    (dict(), 1),
    (dict(), 64),
    (dict(d=2048, num_experts=256, top_k=8), 16),
    (dict(router_weight_bits=8, router_kind=capi.ROUTER_SIGMOID, routed_scaling=2.446, shared_gated=False), 9),
])
def test_static_router_equals_the_handle_router_twice_in_a_row(cuda_device, kw, T):
    layer = Layer(small_config(**kw))
    d = layer.cfg.d
    for call in range(2):  # the second call reuses the array the first one left behind
        a, b = route_both(layer, inputs(T, d, seed=100 + call))
        assert (a[0] == b[0]).all(), "ids differ"
        assert (a[1] == b[1]).all(), "weights differ"
        if a[2] is not None:
            assert (a[2] == b[2]).all(), "shared gate differs"
    layer.close()


def test_static_router_matches_the_oracle_and_leaves_free_memory_alone(cuda_device):
    """The property in the entry point's name: repeated calls change neither the device's free memory
    (cudaMemGetInfo) nor torch's allocator statistics, and the answers are the oracle's, bit for bit."""
    layer = Layer(small_config(d=256, num_experts=64, top_k=8))
    cfg = layer.cfg
    x = inputs(32, cfg.d, seed=7)
    x_dev = to_act_tensor(x, cfg.act_dtype, layer.device)
    ids = torch.zeros((32, 8), dtype=torch.int32, device=layer.device)
    w = torch.zeros((32, 8), dtype=torch.float32, device=layer.device)
    g = torch.zeros(32, dtype=torch.float32, device=layer.device)
    encode_router_static(cfg, layer.router_ops, x_dev, ids, w, g)   # the first call looks the array's address up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0 = torch.cuda.memory_reserved()
    for _ in range(5):
        encode_router_static(cfg, layer.router_ops, x_dev, ids, w, g)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0 and torch.cuda.memory_reserved() == reserved0
    ids_ref, w_ref, _ = layer.oracle_route(x)
    assert (ids.cpu().numpy().astype(np.uint32) == ids_ref).all()
    assert (w.cpu().numpy() == w_ref).all()
    layer.close()


def test_static_router_asks_for_the_gate_operands_like_the_handle_call(cuda_device):
    layer = Layer(small_config())   # shared_gated
    x_dev = to_act_tensor(inputs(2, 128, seed=1), layer.cfg.act_dtype, layer.device)
    ids = torch.zeros((2, 4), dtype=torch.int32, device=layer.device)
    w = torch.zeros((2, 4), dtype=torch.float32, device=layer.device)
    with pytest.raises(ShrikeError) as e:
        encode_router_static(layer.cfg, layer.router_ops, x_dev, ids, w, None)
    assert e.value.code == capi.EINVAL and "shared_gate" in str(e.value)
    with pytest.raises(ShrikeError) as e:   # an offset view: 4-byte aligned only
        base = torch.zeros(2 * 128 + 4, dtype=torch.float32, device=layer.device)
        g = torch.zeros(2, dtype=torch.float32, device=layer.device)
        encode_router_static(layer.cfg, layer.router_ops, base[1:1 + 256].view(2, 128), ids, w, g)
    assert e.value.code == capi.EINVAL and "aligned" in str(e.value)
    layer.close()


def test_static_router_refuses_what_its_array_cannot_hold(cuda_device):
    layer = Layer(small_config(max_tokens=128))
    x_dev = to_act_tensor(inputs(65, 128, seed=1), layer.cfg.act_dtype, layer.device)
    ids = torch.zeros((65, 4), dtype=torch.int32, device=layer.device)
    w = torch.zeros((65, 4), dtype=torch.float32, device=layer.device)
    g = torch.zeros(65, dtype=torch.float32, device=layer.device)
    with pytest.raises(ShrikeError) as e:
        encode_router_static(layer.cfg, layer.router_ops, x_dev, ids, w, g)
    assert e.value.code == capi.ERANGE and "64" in str(e.value)
    layer.close()
