"""The benchmark workloads at their full layer shapes, against the oracle on the
expert blocks the routing actually touches (downloaded from the device pool)."""
import numpy as np
import pytest

from gpu_harness import Layer, inputs, rel_l2
from shrike_b200 import capi
import fixtures as fx

pytestmark = pytest.mark.gpu

TOL = 1e-3


def run(layer: Layer, x, tol=TOL, **kw):
    y, ids, w, _ = layer.forward(x, **kw)
    ids_ref, w_ref, logits = layer.oracle_route(x)
    assert (ids == ids_ref).all() and (w == w_ref).all()
    y_ref = layer.oracle_forward(x, ids_ref, w_ref)
    err = rel_l2(y, y_ref)
    assert err <= tol, f"relative L2 {err:.3e}"
    # how close the routing came to a flip: gap between the k-th and (k+1)-th score
    srt = np.sort(logits, axis=1)[:, ::-1]
    k = layer.cfg.top_k
    return err, float((srt[:, k - 1] - srt[:, k]).min())


@pytest.mark.parametrize("T", [1, 4, 16])
def test_qwen_layer_decode(cuda_device, T):
    """Single MoE layer, Qwen3.5-35B-A3B shape: block 1,769,472 B, top-8 of 256 + gated shared expert."""
    cfg = fx.qwen_config(max_tokens=16, act_dtype=capi.DTYPE_FP32)
    layer = Layer(cfg, seed=101, device_fill=True)
    assert layer.block_bytes == 1_769_472
    err, gap = run(layer, inputs(T, cfg.d, seed=T))
    err2, _ = run(layer, inputs(T, cfg.d, seed=T), fused=True)
    print(f"qwen T={T}: rel L2 {err:.2e} (fused {err2:.2e}), min top-k gap {gap:.2e}")
    layer.close()


@pytest.mark.parametrize("T", [1, 4])
def test_qwen_layer_bf16_in_fp32_out(cuda_device, T):
    """The benchmarked configuration: bf16 x in, fp32 accumulate, fp32 y out, at the stated 1e-3 bar."""
    cfg = fx.qwen_config(max_tokens=16)
    assert cfg.act_dtype == capi.DTYPE_BF16 and cfg.out_dtype == capi.DTYPE_FP32
    layer = Layer(cfg, seed=102, device_fill=True)
    run(layer, inputs(T, cfg.d, seed=9))
    run(layer, inputs(T, cfg.d, seed=9), fused=True)
    layer.close()


def test_qwen_layer_fp16_meta(cuda_device):
    cfg = fx.qwen_config(max_tokens=16, meta_dtype=capi.DTYPE_FP16)
    layer = Layer(cfg, seed=102, device_fill=True)
    run(layer, inputs(2, cfg.d, seed=9))
    layer.close()


@pytest.mark.parametrize("group,T", [(32, 1), (32, 64), (64, 1)])
def test_gpt_oss_layer(cuda_device, group, T):
    """gpt-oss-20B shape: D = F = 2880, 32 experts top-4, additive biases, clamped SwiGLU, no shared expert."""
    cfg = fx.gpt_oss_config(max_tokens=64, group_size=group, act_dtype=capi.DTYPE_FP32)
    layer = Layer(cfg, seed=103, device_fill=True)
    assert layer.block_bytes == (15_569_280 if group == 32 else 14_014_080)
    err, gap = run(layer, inputs(T, cfg.d, seed=group + T))
    run(layer, inputs(T, cfg.d, seed=group + T), fused=True)
    print(f"gpt-oss g{group} T={T}: rel L2 {err:.2e}, min top-k gap {gap:.2e}")
    layer.close()


def test_kimi_layer_decode_and_prefill(cuda_device):
    """Kimi-Linear shape: int8 g64, sigmoid router x2.446 with a selection-only bias, ungated shared expert."""
    rng = np.random.default_rng(5)
    cfg = fx.kimi_config(max_tokens=512, act_dtype=capi.DTYPE_FP32)
    layer = Layer(cfg, seed=104, device_fill=True, logit_bias=rng.uniform(-0.1, 0.1, 256).astype(np.float32))
    assert layer.block_bytes == 7_520_256
    run(layer, inputs(16, cfg.d, seed=1))
    run(layer, inputs(16, cfg.d, seed=1), fused=True)
    run(layer, inputs(96, cfg.d, seed=2), prefill=True)
    layer.close()


def test_qwen_prefill_zipf_chunk(cuda_device):
    """A slice of the ragged prefill workload: Zipf(1.1) prior on the router logits."""
    cfg = fx.qwen_config(max_tokens=256, act_dtype=capi.DTYPE_FP32)
    layer = Layer(cfg, seed=105, device_fill=True, logit_bias=fx.zipf_logit_bias(256, 1.1))
    y, ids, w, _ = layer.forward(inputs(160, cfg.d, seed=3), prefill=True)
    counts = np.bincount(ids.ravel(), minlength=256)
    assert counts.max() >= 20 * max(1, np.median(counts[counts > 0]))
    run(layer, inputs(160, cfg.d, seed=3), prefill=True)
    layer.close()


def sample_rows(T: int, n: int, seed: int) -> np.ndarray:
    return np.sort(np.random.default_rng(seed).choice(T, size=min(n, T), replace=False))


def test_qwen_prefill_full_chunk_4096_rows(cuda_device):
    """The ragged prefill workload at its full size: 4096 bf16 rows, Zipf(1.1) prior, top-8 of 256, on the
    tcgen05 path. Routing of every row is checked bit for bit; y against the oracle on a seeded sample of
    512 rows (the CPU FFN costs about 10 ms per row) plus the 16 rows routed to the most loaded expert."""
    T = 4096
    cfg = fx.qwen_config(max_tokens=T)
    layer = Layer(cfg, seed=107, device_fill=True, logit_bias=fx.zipf_logit_bias(256, 1.1))
    x = inputs(T, cfg.d, seed=41)
    y, ids, w, _ = layer.forward(x, prefill=True)
    ids_ref, w_ref, _ = layer.oracle_route(x)
    assert (ids == ids_ref).all() and (w == w_ref).all()
    counts = np.bincount(ids.ravel(), minlength=256)
    assert counts.max() > 1500 and (counts > 0).sum() > 100   # a few experts take thousands of rows
    busiest = np.where((ids == counts.argmax()).any(axis=1))[0][:16]
    rows = np.unique(np.concatenate([sample_rows(T, 512, 7), busiest]))
    y_ref = layer.oracle_forward(x, ids_ref, w_ref, rows=rows)
    err = rel_l2(y[rows], y_ref)
    assert err <= TOL, f"relative L2 {err:.3e}"
    assert np.isfinite(y).all() and np.abs(y).max() < 1e3
    print(f"qwen prefill 4096 rows: rel L2 {err:.2e} on {rows.size} sampled rows, busiest expert {counts.max()} rows")
    layer.close()


def test_gpt_oss_64_rows_on_the_expert_grouped_path(cuda_device):
    """gpt-oss shape, g32, 64 rows on a handle that owns the prefill operands (max_tokens = 128): the layer
    call takes the tcgen05 path with scale rows of 90 groups (not whole 16-byte units: read by the converter
    threads) at D = F = 2880."""
    cfg = fx.gpt_oss_config(max_tokens=128, group_size=32)
    layer = Layer(cfg, seed=108, device_fill=True)
    err, gap = run(layer, inputs(64, cfg.d, seed=43), fused=True)
    print(f"gpt-oss g32 64 rows, grouped path: rel L2 {err:.2e}, min top-k gap {gap:.2e}")
    layer.close()


def test_layer_forward_host_round_trip(cuda_device):
    """The host-buffer entry point gives what the device-pointer calls give."""
    import torch
    cfg = fx.qwen_config(max_tokens=16, act_dtype=capi.DTYPE_FP32, d=512, f=256, shared_f=256, num_experts=64)
    layer = Layer(cfg, seed=106, device_fill=True)
    x = inputs(5, cfg.d, seed=4)
    y_dev, ids_dev, w_dev, _ = layer.forward(x)
    x_host = torch.from_numpy(x.copy())
    y_host = torch.empty_like(x_host)
    ids_host = torch.zeros((5, 8), dtype=torch.int32)
    w_host = torch.zeros((5, 8), dtype=torch.float32)
    layer.moe.layer_forward_host(layer.pool, layer.offsets, 0, layer.router_ops, x_host, y_host, layer.shared,
                                 ids_host, w_host)
    assert (y_host.numpy() == y_dev).all()
    assert (ids_host.numpy().astype(np.uint32) == ids_dev).all() and (w_host.numpy() == w_dev).all()
    layer.close()


@pytest.mark.parametrize("T", [1, 3])
def test_decode_stack_host_entry_point_equals_the_layer_calls(cuda_device, T):
    """shrike_decode_stack_forward_host (host rows in, every layer, host rows out) against the same layers called
    one by one with device pointers, and the first layer's output against the oracle. Three stacked layers that
    share one pool; the residual stream takes a fresh row before every layer."""
    import torch
    from shrike_b200.moe import DecodeStack
    cfg = fx.qwen_config(max_tokens=16, d=512, f=256, shared_f=256, num_experts=64, y_dtype=capi.DTYPE_FP32)
    layers = [Layer(cfg, seed=150 + l, device_fill=True) for l in range(3)]
    # block 0 enters layer 0; block l + 1 is what layer l's output is added to and what layer l + 1 reads
    rows = np.stack([fx.round_bf16(inputs(T, cfg.d, seed=60 + l)) for l in range(4)])
    rows_host = torch.from_numpy(rows).to(torch.bfloat16).contiguous()
    out_host = torch.empty((T, cfg.d), dtype=torch.bfloat16)
    stack = DecodeStack([(L.moe, L.pool, L.offsets, 0, L.router_ops, L.shared) for L in layers], T)
    for _ in range(2):   # a second call reuses every buffer
        stack.forward_host(rows_host, out_host)
    for L in layers:
        L.moe.status()
    # the same stream, layer by layer
    dev = torch.device("cuda:0")
    blocks = rows_host.to(dev)
    y = torch.empty((T, cfg.d), dtype=torch.float32, device=dev)
    ids = torch.zeros((T, cfg.top_k), dtype=torch.int32, device=dev)
    w = torch.zeros((T, cfg.top_k), dtype=torch.float32, device=dev)
    for l, L in enumerate(layers):
        L.moe.encode_decode_layer(L.pool, L.offsets, 0, L.router_ops, blocks[l], y, blocks[l + 1], L.shared, ids, w)
        if l == 0:
            torch.cuda.synchronize()
            y0, ids0, w0 = y.cpu().numpy().copy(), ids.cpu().numpy().astype(np.uint32), w.cpu().numpy().copy()
    torch.cuda.synchronize()
    assert torch.equal(out_host, blocks[3].cpu())
    ids_ref, w_ref, _ = layers[0].oracle_route(rows[0])
    assert (ids0 == ids_ref).all() and (w0 == w_ref).all()
    assert rel_l2(y0, layers[0].oracle_forward(rows[0], ids_ref, w_ref)) <= TOL
    stack.close()
    for L in layers:
        L.close()
