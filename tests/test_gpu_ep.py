"""Expert parallelism on GPUs: the CUDA dispatch/combine kernels against the numpy protocol, and the
whole expert-parallel layer against the oracle -- with one rank always, with two NCCL ranks when the box
has two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _config(ne=16, act=None):
    from shrike_b200 import capi
    from shrike_b200.moe import MoEConfig
    return MoEConfig(d=256, f=128, num_experts=ne, top_k=4, act_dtype=capi.DTYPE_FP32 if act is None else act,
                     has_shared=True, shared_gated=False, shared_f=128, max_tokens=256)


def _problem(T, cfg, seed=5):
    import fixtures as fx
    rng = np.random.default_rng(seed)
    x = fx.round_bf16(rng.normal(0, 1, (T, cfg.d)).astype(np.float32))
    router = rng.normal(0, 0.05, (cfg.num_experts, cfg.d)).astype(np.float32)
    return x, router


def _oracle(cfg, x, router, seed):
    import oracle_lib as O
    import fixtures as fx
    T = x.shape[0]
    ids = np.zeros((T, cfg.top_k), np.uint32)
    w = np.zeros((T, cfg.top_k), np.float32)
    for t in range(T):
        ids[t], w[t] = O.router_select(O.router_logits_f32(router, x[t]), cfg.top_k, round_f16=True)
    ecfg = O.expert_cfg(cfg.d, cfg.f)
    blocks = {int(e): fx.synth_block(cfg, seed, 0, int(e)) for e in np.unique(ids)}
    shared = fx.synth_block(cfg, seed, 0, 100000, shared=True)
    y = O.moe_layer(O.layer_cfg(ecfg, O.expert_cfg(cfg.d, cfg.shared_f), False), blocks, shared, None, x, ids, w)
    return ids, w, y


def _run_rank(rank, world, port, T, seed, out_path):
    """One EP rank: builds its shard, runs the layer on its rows, saves y."""
    import torch.distributed as dist
    from shrike_b200 import capi
    import fixtures as fx
    from shrike_b200.ep import ExpertParallelLayer
    from shrike_b200.moe import RouterOperands, expert_offsets
    cfg = _config()
    torch.cuda.set_device(rank)
    group = None
    if world > 1:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    x, router = _problem(T, cfg)
    per = T // world
    layer = ExpertParallelLayer(cfg, rank, world, rank, per, group)
    for e in range(layer.lo, layer.hi):
        layer.pool.upload(e - layer.lo, fx.synth_block(cfg, seed, 0, e))
    dev = torch.device("cuda", rank)
    sh = torch.from_numpy(fx.synth_block(cfg, seed, 0, 100000, shared=True).copy()).to(dev)
    layer.set_shared(capi.SharedExpert(sh.data_ptr(), expert_offsets(cfg, shared=True)[0]))
    ops = RouterOperands(weights=torch.from_numpy(router).to(dev))
    xl = torch.from_numpy(x[rank * per:(rank + 1) * per].copy()).to(dev)
    y = torch.empty_like(xl)
    h = xl.clone()
    for _ in range(2):  # a second pass reuses every buffer
        h.copy_(xl)
        layer.forward(ops, xl, y, h)
    layer.home.status()
    layer.routed.status()
    np.save(out_path, np.stack([y.cpu().numpy(), h.cpu().numpy()]))
    ids = layer.ids.cpu().numpy().astype(np.uint32)
    np.save(out_path + ".pack.npy", np.concatenate([layer.send_counts.cpu().numpy().astype(np.int64),
                                                    layer.row_of.cpu().numpy().astype(np.int64).ravel()]))
    np.save(out_path + ".ids.npy", ids)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    layer.close()


@pytest.mark.parametrize("T", [8, 96])
def test_single_rank_expert_parallel_layer(cuda_device, tmp_path, T):
    seed = 21
    out = str(tmp_path / "y0.npy")
    _run_rank(0, 1, 0, T, seed, out)
    cfg = _config()
    x, router = _problem(T, cfg)
    ids, w, y_ref = _oracle(cfg, x, router, seed)
    got = np.load(out)
    assert (np.load(out + ".ids.npy") == ids).all()
    assert np.linalg.norm(got[0] - y_ref) / np.linalg.norm(y_ref) <= 1e-3
    assert np.abs(got[1] - (x + got[0])).max() <= 1e-5 * np.abs(x).max()


def test_cuda_dispatch_matches_the_protocol(cuda_device, tmp_path):
    import ep_reference as R
    T, seed = 96, 22
    out = str(tmp_path / "y0.npy")
    _run_rank(0, 1, 0, T, seed, out)
    cfg = _config()
    x, router = _problem(T, cfg)
    ids, w, _ = _oracle(cfg, x, router, seed)
    # the same rows packed for an imagined 4-rank world, through the C ABI
    from shrike_b200.moe import MoE, _ptr, _stream
    import dataclasses
    moe = MoE(dataclasses.replace(cfg, max_tokens=T))
    dev = torch.device("cuda:0")
    world, epr, cap = 4, cfg.num_experts // 4, T
    xd = torch.from_numpy(x).to(dev)
    idd = torch.from_numpy(ids.astype(np.int32)).to(dev)
    wd = torch.from_numpy(w).to(dev)
    sx = torch.zeros((world, cap, cfg.d), dtype=torch.float32, device=dev)
    si = torch.zeros((world, cap, cfg.top_k), dtype=torch.int32, device=dev)
    sw = torch.zeros((world, cap, cfg.top_k), dtype=torch.float32, device=dev)
    sc = torch.zeros(world, dtype=torch.int32, device=dev)
    ro = torch.zeros((T, world), dtype=torch.int32, device=dev)
    moe._check(moe._lib.shrike_ep_encode_dispatch(moe._h, _stream(), _ptr(xd), _ptr(idd), _ptr(wd), T, world, epr, cap,
                                                  _ptr(sx), _ptr(si), _ptr(sw), _ptr(sc), _ptr(ro)))
    moe.status()
    rx, ri, rw, rc, rr = R.pack(x, ids, w, world, epr, cap)
    assert (sc.cpu().numpy() == rc).all() and (ro.cpu().numpy() == rr).all()
    assert (si.cpu().numpy().astype(np.uint32) == ri).all()
    for g in range(world):
        n = int(rc[g])
        assert (sx.cpu().numpy()[g, :n] == rx[g, :n]).all() and (sw.cpu().numpy()[g, :n] == rw[g, :n]).all()
    moe.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_nccl_ranks_match_the_oracle(cuda_device, tmp_path):
    import subprocess
    T, seed, world = 96, 23, 2
    port = _free_port()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(world):
        code = (f"import sys; sys.path.insert(0, {root!r}); sys.path.insert(0, {root + '/tests'!r}); "
                f"import test_gpu_ep as t; t._run_rank({r}, {world}, {port}, {T}, {seed}, {str(tmp_path / f'y{r}.npy')!r})")
        procs.append(subprocess.Popen([sys.executable, "-c", code]))
    for p in procs:
        assert p.wait(timeout=300) == 0
    cfg = _config()
    x, router = _problem(T, cfg)
    ids, w, y_ref = _oracle(cfg, x, router, seed)
    y = np.concatenate([np.load(str(tmp_path / f"y{r}.npy"))[0] for r in range(world)])
    assert np.linalg.norm(y - y_ref) / np.linalg.norm(y_ref) <= 1e-3
