"""Expert parallelism, host-side protocol on CPU: two gloo ranks exchange packed rows, run their own
experts (the oracle stands in for the GPU kernels here) and combine; the result must equal the
single-process layer. Covers the N > 1 logic without a GPU."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _layer_inputs():
    import oracle_lib as O
    import fixtures as fx
    d, f, ne, k, T = 128, 64, 8, 2, 12
    rng = np.random.default_rng(3)
    x = fx.round_bf16(rng.normal(0, 1, (T, d)).astype(np.float32))
    router = rng.normal(0, 0.05, (ne, d)).astype(np.float32)
    ecfg = O.expert_cfg(d, f)
    blocks = {e: O.synth_block(ecfg, 11, 0, e) for e in range(ne)}
    shared = O.synth_block(ecfg, 11, 0, 100000)
    ids = np.zeros((T, k), np.uint32)
    w = np.zeros((T, k), np.float32)
    for t in range(T):
        ids[t], w[t] = O.router_select(O.router_logits_f32(router, x[t]), k, round_f16=True)
    return d, f, ne, k, T, x, ids, w, blocks, shared, ecfg


def _rank_main(rank, world, port, out):
    import oracle_lib as O
    import ep_reference as R
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    d, f, ne, k, T, x, ids, w, blocks, shared, ecfg = _layer_inputs()
    per = T // world
    epr = ne // world
    lo = rank * per
    xl, il, wl = x[lo:lo + per], ids[lo:lo + per], w[lo:lo + per]
    cap = per
    send_x, send_ids, send_w, counts, row_of = R.pack(xl, il, wl, world, epr, cap)

    def a2a(a):
        t_in = torch.from_numpy(np.ascontiguousarray(a)).view(-1)
        t_out = torch.empty_like(t_in)
        dist.all_to_all_single(t_out, t_in)
        return t_out.numpy().reshape(a.shape)

    recv_x, recv_ids, recv_w = a2a(send_x), a2a(send_ids.view(np.int32)).view(np.uint32), a2a(send_w)
    # local experts on every received row; invalid ids get weight 0 and a valid dummy id
    rows = world * cap
    rid = recv_ids.reshape(rows, k)
    valid = rid != R.INVALID
    gid = np.where(valid, rid + rank * epr, rank * epr).astype(np.uint32)
    rw = np.where(valid, recv_w.reshape(rows, k), 0).astype(np.float32)
    y_part = O.moe_layer(O.layer_cfg(ecfg), {e: blocks[e] for e in range(rank * epr, (rank + 1) * epr)}, None, None,
                         recv_x.reshape(rows, d), gid, rw)
    back = a2a(y_part.reshape(world, cap, d))
    y_home = O.moe_layer(O.layer_cfg(ecfg, ecfg, False), {0: blocks[0]}, shared, None, xl,
                         np.zeros((per, k), np.uint32), np.zeros((per, k), np.float32))
    y = R.combine(back, row_of, y_home)
    out[rank] = (y, counts.copy(), row_of.copy())
    dist.barrier()
    dist.destroy_process_group()


def _spawn_target(rank, world, port, queue):
    out = {}
    _rank_main(rank, world, port, out)
    queue.put((rank, out[rank]))


def test_two_gloo_ranks_reproduce_the_single_process_layer():
    import oracle_lib as O
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_spawn_target, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    d, f, ne, k, T, x, ids, w, blocks, shared, ecfg = _layer_inputs()
    y_ref = O.moe_layer(O.layer_cfg(ecfg, ecfg, False), blocks, shared, None, x, ids, w)
    y = np.concatenate([results[r][0] for r in range(world)])
    assert np.abs(y - y_ref).max() <= 1e-5 * max(1.0, np.abs(y_ref).max())
    # every (row, rank) with an expert there was sent exactly once
    per = T // world
    for r in range(world):
        counts, row_of = results[r][1], results[r][2]
        dest = ids[r * per:(r + 1) * per] // (ne // world)
        for g in range(world):
            assert counts[g] == sum((dest[t] == g).any() for t in range(per))
            sent = sorted(int(v) for v in row_of[:, g] if v >= 0)
            assert sent == list(range(int(counts[g])))


def test_pack_reference_rows_are_in_token_order_and_bounded():
    import ep_reference as R
    ids = np.array([[0, 5], [6, 7], [1, 2], [4, 3]], dtype=np.uint32)
    w = np.arange(8, dtype=np.float32).reshape(4, 2)
    x = np.arange(4 * 3, dtype=np.float32).reshape(4, 3)
    sx, si, sw, counts, row_of = R.pack(x, ids, w, 2, 4, 4)
    assert list(counts) == [3, 3]
    assert row_of.tolist() == [[0, 0], [-1, 1], [1, -1], [2, 2]]
    assert si[0, 0].tolist() == [0, R.INVALID] and si[1, 0].tolist() == [R.INVALID, 1]
    assert sw[1, 1].tolist() == [2.0, 3.0] and (sx[0, 2] == x[3]).all()
