"""The C++ host mirror (shrike_b200/host/shrike_moe.hpp): compiles against the C ABI, and a C++ host that
encodes one routed layer in the reference runner's call order gets the oracle's answer."""
import subprocess
import tempfile
from pathlib import Path

import numpy as np
import pytest

from shrike_b200 import build


def test_cpp_host_mirror_compiles_and_links():
    exe = build.build_harness()
    assert exe.exists()
    # wrong usage is an ordinary exit code, not a crash
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 64 and "usage" in res.stderr


@pytest.mark.gpu
def test_cpp_host_runs_the_layer_like_the_oracle(cuda_device):
    import oracle_lib as O
    from shrike_b200 import capi
    import fixtures as fx
    from shrike_b200.moe import MoEConfig

    exe = build.build_harness()
    seed, rows = 4242, 5
    cfg = MoEConfig(d=512, f=256, num_experts=32, top_k=8, act_dtype=capi.DTYPE_FP32, has_shared=True,
                    shared_gated=True, shared_f=256, max_tokens=16)
    rng = np.random.default_rng(7)
    router = rng.normal(0, 0.02, (32, 512)).astype(np.float32)
    gate = rng.normal(0, 0.02, 512).astype(np.float32)
    x = fx.round_bf16(rng.normal(0, 1, (rows, 512)).astype(np.float32))
    with tempfile.TemporaryDirectory() as tmp:
        out = Path(tmp) / "out.bin"
        res = subprocess.run([str(exe), str(seed), str(rows), str(out)],
                             input=np.concatenate([router.ravel(), gate, x.ravel()]).astype(np.float32).tobytes(),
                             capture_output=True)
        assert res.returncode == 0, res.stderr.decode()
        raw = np.fromfile(out, dtype=np.uint32)
    ids = raw[:rows * 8].reshape(rows, 8)
    y = raw[rows * 8:rows * 8 + rows * 512].view(np.float32).reshape(rows, 512)
    y2 = raw[rows * 8 + rows * 512:].view(np.float32).reshape(rows, 512)
    ids_ref = np.zeros_like(ids)
    w_ref = np.zeros((rows, 8), dtype=np.float32)
    for t in range(rows):
        ids_ref[t], w_ref[t] = O.router_select(O.router_logits_f32(router, x[t]), 8, round_f16=True)
    assert (ids == ids_ref).all()
    ecfg = O.expert_cfg(512, 256)
    blocks = {int(e): fx.synth_block(cfg, seed, 0, int(e)) for e in np.unique(ids_ref)}
    shared = fx.synth_block(cfg, seed, 0, 100000, shared=True)
    y_ref = O.moe_layer(O.layer_cfg(ecfg, ecfg, True), blocks, shared, gate, x, ids_ref, w_ref)
    err = np.linalg.norm(y - y_ref) / np.linalg.norm(y_ref)
    assert err <= 1e-3, err
    assert (y == y2).all(), "the one-call layer and the five separate encodes differ"
