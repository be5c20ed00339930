"""Expert parallelism on GPUs: the expert-parallel layer against the oracle -- over peer memory (the C ABI's
shrike_ep_*) and over NCCL all-to-all (the checker) -- with one rank always, with two ranks when the box has
two GPUs; the pack kernel against the numpy protocol; the full-size mixed batch; and a wait that runs out
because nothing ever writes its word (a peer that never answers, made on the host)."""
import dataclasses
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


def _build_layer(cfg, rank, world, per, seed, exchange, group=None):
    from shrike_b200 import capi
    import fixtures as fx
    from shrike_b200.ep import ExpertParallelLayer
    from shrike_b200.moe import expert_offsets
    layer = ExpertParallelLayer(cfg, rank, world, rank if torch.cuda.device_count() > rank else 0, per, group,
                                exchange=exchange)
    for e in range(layer.lo, layer.hi):
        layer.pool.upload(e - layer.lo, fx.synth_block(cfg, seed, 0, e))
    sh = torch.from_numpy(fx.synth_block(cfg, seed, 0, 100000, shared=True).copy()).to(layer.dev)
    layer._shared_block = sh
    layer.set_shared(capi.SharedExpert(sh.data_ptr(), expert_offsets(cfg, shared=True)[0]))
    return layer


def _run_rank(rank, world, port, T, seed, out_path, exchange="peer"):
    """One EP rank: builds its shard, runs the layer twice on its rows, saves y, hidden and the routing."""
    import torch.distributed as dist
    from shrike_b200.moe import RouterOperands
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
    layer = _build_layer(cfg, rank, world, per, seed, exchange, group)
    dev = layer.dev
    ops = RouterOperands(weights=torch.from_numpy(router).to(dev))
    xl = torch.from_numpy(x[rank * per:(rank + 1) * per].copy()).to(dev)
    y = torch.empty_like(xl)
    h = xl.clone()
    for _ in range(2):  # a second pass reuses every buffer
        h.copy_(xl)
        layer.forward(ops, xl, y, h)
    layer.status()
    np.save(out_path, np.stack([y.cpu().numpy(), h.cpu().numpy()]))
    ids, _ = layer.routing(ops, xl)
    np.save(out_path + ".ids.npy", ids.cpu().numpy().astype(np.uint32))
    if exchange == "peer":
        sent, received, nbytes = layer.last_counts()
        np.save(out_path + ".counts.npy", np.array(sent + [received, nbytes], dtype=np.int64))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    layer.close()


@pytest.mark.parametrize("exchange", ["peer", "nccl"])
@pytest.mark.parametrize("T", [8, 96])
def test_single_rank_expert_parallel_layer(cuda_device, tmp_path, T, exchange):
    seed = 21
    out = str(tmp_path / "y0.npy")
    _run_rank(0, 1, 0, T, seed, out, exchange)
    cfg = _config()
    x, router = _problem(T, cfg)
    ids, w, y_ref = _oracle(cfg, x, router, seed)
    got = np.load(out)
    assert (np.load(out + ".ids.npy") == ids).all()
    assert np.linalg.norm(got[0] - y_ref) / np.linalg.norm(y_ref) <= 1e-3
    assert np.abs(got[1] - (x + got[0])).max() <= 1e-5 * np.abs(x).max()
    if exchange == "peer":
        counts = np.load(out + ".counts.npy")
        assert counts[0] == T and counts[1] == T   # every row has a pick on the only rank; nothing leaves it
        assert counts[2] == 0


def test_cuda_dispatch_matches_the_protocol(cuda_device):
    import ep_reference as R
    T, seed = 96, 22
    cfg = _config()
    x, router = _problem(T, cfg)
    ids, w, _ = _oracle(cfg, x, router, seed)
    # the rows packed for an imagined 4-rank world, through the C ABI
    from shrike_b200.moe import MoE, _ptr, _stream
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


def test_full_size_mixed_batch_on_one_rank(cuda_device):
    """The expert-parallel workload at its full per-rank size: 16 decode rows + one 2048-row prefill chunk of the
    Kimi-Linear shape (int8 g64, 256 experts top-8 sigmoid with a selection bias, shared expert), bf16 rows in,
    fp32 rows out, through the peer-memory layer with every expert on this rank; sampled rows against the oracle."""
    import fixtures as fx
    import oracle_lib as O
    from shrike_b200 import capi
    from shrike_b200.ep import ExpertParallelLayer
    from shrike_b200.moe import RouterOperands, expert_offsets
    from gpu_harness import bf16_tensor
    rows, seed = 16 + 2048, 31
    cfg = fx.kimi_config(max_tokens=rows)
    dev = torch.device("cuda:0")
    layer = ExpertParallelLayer(cfg, 0, 1, 0, rows)
    layer.pool.fill_synthetic(0, layer.epr, seed, 0, first_expert=0)
    soff, _ = expert_offsets(cfg, shared=True)
    sh = torch.from_numpy(fx.synth_block(cfg, seed, 0, 100000, shared=True).copy()).to(dev)
    layer.set_shared(capi.SharedExpert(sh.data_ptr(), soff))
    rng = np.random.default_rng(seed)
    router = rng.normal(0, 0.05, (cfg.num_experts, cfg.d)).astype(np.float32)
    correction = rng.uniform(-0.1, 0.1, cfg.num_experts).astype(np.float32)
    xr = fx.round_bf16(rng.normal(0, 1, (rows, cfg.d)).astype(np.float32))
    ops = RouterOperands(weights=torch.from_numpy(router).to(dev), logit_bias=bf16_tensor(correction, dev))
    x = torch.from_numpy(xr).to(torch.bfloat16).to(dev)
    y = torch.empty((rows, cfg.d), dtype=torch.float32, device=dev)
    layer.forward(ops, x, y)
    layer.status()
    ids, w = layer.routing(ops, x)
    ids, w = ids.cpu().numpy().astype(np.uint32), w.cpu().numpy()
    assert all(len(set(r)) == cfg.top_k for r in ids[:64].tolist())
    sample = np.sort(rng.choice(rows, 40, replace=False))
    ecfg = O.expert_cfg(cfg.d, cfg.f, bits=8)
    lcfg = O.layer_cfg(ecfg, O.expert_cfg(cfg.d, cfg.shared_f, bits=8), False)
    blocks = {int(e): fx.synth_block(cfg, seed, 0, int(e)) for e in np.unique(ids[sample])}
    ref = O.moe_layer(lcfg, blocks, fx.synth_block(cfg, seed, 0, 100000, shared=True), None, xr[sample], ids[sample],
                      w[sample], threads=os.cpu_count() or 8)
    got = y.cpu().numpy()[sample]
    assert np.isfinite(y.cpu().numpy()).all()
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-3
    sent, received, nbytes = layer.last_counts()
    assert sent[0] == rows and received == rows and nbytes == 0
    layer.close()


def test_a_peer_that_never_answers_ends_in_a_timeout_status(cuda_device):
    """Rank 0 of an imagined two-rank world whose peer buffer is plain memory that nothing writes: the bounded
    waits for the peer's arrival words run out, the call returns, and the status says timeout. No GPU fault, no
    second process: the failure is made on the host by never starting the peer."""
    from shrike_b200 import capi
    from shrike_b200.ep import ExpertParallelLayer
    from shrike_b200.moe import RouterOperands, ShrikeError, expert_offsets
    cfg = _config()
    T, seed = 32, 24
    x, router = _problem(T, cfg)
    dev = torch.device("cuda:0")
    layer = ExpertParallelLayer(cfg, 0, 2, 0, T, None, exchange="peer", connect=False)
    base, nbytes = layer.buffer()
    fake_peer = torch.zeros(nbytes, dtype=torch.uint8, device=dev)   # the peer that never runs
    layer.connect_pointers([base, fake_peer.data_ptr()])
    layer.set_wait_polls(200)   # a fraction of a millisecond per wait
    import fixtures as fx
    for e in range(layer.lo, layer.hi):
        layer.pool.upload(e - layer.lo, fx.synth_block(cfg, seed, 0, e))
    sh = torch.from_numpy(fx.synth_block(cfg, seed, 0, 100000, shared=True).copy()).to(dev)
    layer.set_shared(capi.SharedExpert(sh.data_ptr(), expert_offsets(cfg, shared=True)[0]))
    ops = RouterOperands(weights=torch.from_numpy(router).to(dev))
    xd = torch.from_numpy(x).to(dev)
    y = torch.empty_like(xd)
    layer.forward(ops, xd, y)   # returns: every wait is bounded
    with pytest.raises(ShrikeError) as err:
        layer.status()
    assert err.value.code == capi.ETIMEDOUT
    assert torch.isfinite(y).all()
    # the context is intact: a one-rank layer on the same GPU still answers
    torch.cuda.synchronize()
    layer.close()
    out_ok = torch.zeros(4, device=dev) + 1
    assert float(out_ok.sum()) == 4.0


def _two_ranks(tmp_path, exchange, T=96, seed=23):
    import subprocess
    world = 2
    port = _free_port()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(world):
        code = (f"import sys; sys.path.insert(0, {root!r}); sys.path.insert(0, {root + '/tests'!r}); "
                f"import test_gpu_ep as t; t._run_rank({r}, {world}, {port}, {T}, {seed}, "
                f"{str(tmp_path / f'y{r}.npy')!r}, {exchange!r})")
        procs.append(subprocess.Popen([sys.executable, "-c", code]))
    for p in procs:
        assert p.wait(timeout=300) == 0
    cfg = _config()
    x, router = _problem(T, cfg)
    ids, w, y_ref = _oracle(cfg, x, router, seed)
    y = np.concatenate([np.load(str(tmp_path / f"y{r}.npy"))[0] for r in range(world)])
    assert np.linalg.norm(y - y_ref) / np.linalg.norm(y_ref) <= 1e-3
    return ids


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_over_peer_memory_match_the_oracle(cuda_device, tmp_path):
    ids = _two_ranks(tmp_path, "peer")
    # rows sent: rank r's rows with a pick in each half of the experts
    cfg = _config()
    per = ids.shape[0] // 2
    for r in range(2):
        counts = np.load(str(tmp_path / f"y{r}.npy.counts.npy"))
        mine = ids[r * per:(r + 1) * per]
        for g in range(2):
            assert counts[g] == int(((mine // (cfg.num_experts // 2)) == g).any(axis=1).sum())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_nccl_ranks_match_the_oracle(cuda_device, tmp_path):
    _two_ranks(tmp_path, "nccl")


@pytest.mark.parametrize("T", [8, 96])
def test_int8_shared_expert_beside_int4_routed_experts(cuda_device, T):
    """The reference's Qwen layers keep the shared expert in int8 and the routed experts in int4
    (SharedExpertInt8.swift:55-227): the home handle describes the shared expert's block, the routed handle the
    routed experts'; one rank. Against the oracle with the two formats."""
    import fixtures as fx
    import oracle_lib as O
    from shrike_b200 import capi
    from shrike_b200.ep import ExpertParallelLayer
    from shrike_b200.moe import RouterOperands, expert_offsets
    seed = 27
    cfg4 = _config()                                         # routed experts: int4
    cfg8 = dataclasses.replace(cfg4, weight_bits=8)          # the shared expert's format
    x, router = _problem(T, cfg4)
    dev = torch.device("cuda:0")
    layer = ExpertParallelLayer(cfg8, 0, 1, 0, T, None, exchange="peer", routed_config=cfg4)
    for e in range(layer.lo, layer.hi):
        layer.pool.upload(e - layer.lo, fx.synth_block(cfg4, seed, 0, e))
    sh_block = fx.synth_block(cfg8, seed, 0, 100000, shared=True)
    sh = torch.from_numpy(sh_block.copy()).to(dev)
    layer.set_shared(capi.SharedExpert(sh.data_ptr(), expert_offsets(cfg8, shared=True)[0]))
    ops = RouterOperands(weights=torch.from_numpy(router).to(dev))
    xd = torch.from_numpy(x).to(dev)
    y = torch.empty_like(xd)
    layer.forward(ops, xd, y)
    layer.status()
    ids = np.zeros((T, cfg4.top_k), np.uint32)
    w = np.zeros((T, cfg4.top_k), np.float32)
    for t in range(T):
        ids[t], w[t] = O.router_select(O.router_logits_f32(router, x[t]), cfg4.top_k, round_f16=True)
    blocks = {int(e): fx.synth_block(cfg4, seed, 0, int(e)) for e in np.unique(ids)}
    lcfg = O.layer_cfg(O.expert_cfg(cfg4.d, cfg4.f), O.expert_cfg(cfg4.d, cfg4.shared_f, bits=8), False)
    y_ref = O.moe_layer(lcfg, blocks, sh_block, None, x, ids, w)
    got = y.cpu().numpy()
    assert np.linalg.norm(got - y_ref) / np.linalg.norm(y_ref) <= 1e-3
    layer.close()
