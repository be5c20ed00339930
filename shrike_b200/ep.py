"""Expert-parallel MoE layer: one process per GPU, routed experts sharded over the ranks.

Rank r owns experts [r*NE/G, (r+1)*NE/G). Rows are sharded by home rank; the router and the shared
expert are replicated and run on the home rank. Per layer: route -> dispatch -> local experts -> return ->
combine.

exchange="peer" (default): the whole layer is `shrike_ep_forward` of the C ABI. Rows travel as plain stores
into the destination rank's exchange buffer over NVLink (opened through CUDA IPC handles that this class
passes around with `torch.distributed.all_gather_object`), only the routed rows move, and the shared expert
runs on a second stream beside the exchange. torch.distributed is used once, to hand the 64-byte tokens round.

exchange="nccl": the earlier form, kept as the checker of the peer path -- the library's pack / local-slots /
combine kernels around fixed-capacity `all_to_all_single` calls over the process group.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Optional

import torch
import torch.distributed as dist

from . import capi
from .moe import ExpertCellArena, MoE, MoEConfig, RouterOperands, ShrikeError, _ptr, _stream, expert_offsets, round_up


def shard_range(num_experts: int, world: int, rank: int) -> tuple[int, int]:
    """Experts [lo, hi) owned by `rank` (equal shards; num_experts must divide evenly)."""
    if num_experts % world:
        raise ValueError("num_experts must be a multiple of the world size")
    per = num_experts // world
    return rank * per, (rank + 1) * per


class ExpertParallelLayer:
    """One MoE layer under expert parallelism on this rank's GPU."""

    def __init__(self, config: MoEConfig, rank: int, world: int, device: int, rows_per_rank: int,
                 group: Optional[dist.ProcessGroup] = None, exchange: str = "peer", connect: bool = True,
                 routed_config: Optional[MoEConfig] = None):
        """connect=False (peer exchange, world > 1): the ranks' buffers are not exchanged through the process
        group; the caller hands the peers' base pointers to `connect_pointers` (one process driving several
        GPUs, or a test that stands in for a peer).
        routed_config: the routed experts' weight format where it differs from the shared expert's (`config` then
        describes the shared expert's block: an int8 shared expert beside int4 routed experts); peer exchange only."""
        if exchange not in ("peer", "nccl"):
            raise ValueError("exchange must be 'peer' or 'nccl'")
        self.cfg = config
        self.rank, self.world, self.group, self.exchange = rank, world, group, exchange
        self.rows = rows_per_rank
        self.cap = rows_per_rank  # a row goes to a rank at most once
        self.lo, self.hi = shard_range(config.num_experts, world, rank)
        self.epr = self.hi - self.lo
        self.dev = torch.device("cuda", device)
        # home handle: router over all experts + the shared expert on this rank's rows
        self.home = MoE(dataclasses.replace(config, max_tokens=max(rows_per_rank, 1)), device)
        # routed handle: this rank's experts on every row it may receive
        recv_rows = world * self.cap
        rcfg = routed_config if routed_config is not None else config
        if routed_config is not None and exchange != "peer":
            raise ValueError("routed_config needs the peer exchange")
        self.routed = MoE(dataclasses.replace(rcfg, num_experts=self.epr, has_shared=False, shared_gated=False,
                                              shared_f=0, max_tokens=max(recv_rows, 65)), device)
        self.offsets, self.block_bytes = expert_offsets(rcfg)
        self.pool = ExpertCellArena(self.routed, self.epr, round_up(self.block_bytes, 256))
        self.routed.create_residency(1)
        self.routed.residency_set_layer_identity(0, 0)
        self.shared: Optional[capi.SharedExpert] = None
        self._lib = self.home._lib
        self._ep = None
        k, d = config.top_k, config.d
        T, G, cap = rows_per_rank, world, self.cap
        z = lambda *shape, dtype: torch.zeros(shape, dtype=dtype, device=self.dev)
        if exchange == "peer":
            h = C.c_void_p()
            self.home._check(self._lib.shrike_ep_create(self.home._h, self.routed._h, rank, world, rows_per_rank, C.byref(h)))
            self._ep = h
            if world > 1 and connect:
                token = C.create_string_buffer(capi.EP_HANDLE_BYTES)
                self.home._check(self._lib.shrike_ep_export(self._ep, token))
                tokens = [None] * world
                dist.all_gather_object(tokens, bytes(token.raw), group=group)
                self.home._check(self._lib.shrike_ep_connect(self._ep, b"".join(tokens)))
            # what the peer path keeps inside the library, for callers that look at the routing
            self.ids, self.w = z(T, k, dtype=torch.int32), z(T, k, dtype=torch.float32)
            return
        act, yt = config.torch_act_dtype, config.torch_y_dtype
        self.ids, self.w = z(T, k, dtype=torch.int32), z(T, k, dtype=torch.float32)
        self.gate = z(T, dtype=torch.float32) if config.shared_gated else None
        self.miss_slots = torch.full((T, k), -1, dtype=torch.int32, device=self.dev)
        self.send_x, self.recv_x = z(G, cap, d, dtype=act), z(G, cap, d, dtype=act)
        self.send_ids, self.recv_ids = z(G, cap, k, dtype=torch.int32), z(G, cap, k, dtype=torch.int32)
        self.send_w, self.recv_w = z(G, cap, k, dtype=torch.float32), z(G, cap, k, dtype=torch.float32)
        self.send_counts = z(G, dtype=torch.int32)
        self.row_of = z(T, G, dtype=torch.int32)
        self.slots = z(G * cap, k, dtype=torch.int32)
        self.y_part, self.y_back = z(G * cap, d, dtype=yt), z(G, cap, d, dtype=yt)
        self.y_home = z(T, d, dtype=yt) if config.has_shared else None

    def close(self):
        if self._ep is not None:
            self._lib.shrike_ep_destroy(self._ep)
            self._ep = None
        self.pool.close()
        self.routed.close()
        self.home.close()

    def set_shared(self, shared: capi.SharedExpert) -> None:
        self.shared = shared

    def buffer(self) -> tuple[int, int]:
        """(base address, bytes) of this rank's exchange buffer."""
        base, nbytes = C.c_void_p(), C.c_uint64()
        self.home._check(self._lib.shrike_ep_buffer(self._ep, C.byref(base), C.byref(nbytes)))
        return base.value, nbytes.value

    def connect_pointers(self, bases) -> None:
        """bases[g]: base address of rank g's exchange buffer as this process can address it (own entry ignored)."""
        ptrs = (C.c_void_p * capi.EP_MAX_WORLD)()
        for g, b in enumerate(bases):
            ptrs[g] = b
        self.home._check(self._lib.shrike_ep_connect_pointers(self._ep, ptrs))

    def set_wait_polls(self, polls: int) -> None:
        """Limit of the bounded device-side waits for the peers' arrival words (0 = the default, about a second)."""
        self.home._check(self._lib.shrike_ep_set_wait_polls(self._ep, polls))

    def status(self) -> None:
        """Synchronises the current stream and raises if a kernel of either handle reported a failure."""
        if self._ep is not None:
            rc = self._lib.shrike_ep_status(self._ep, _stream())
            if rc:
                raise ShrikeError(rc, self._lib.shrike_last_error(self.home._h).decode())
        else:
            self.home.status()
            self.routed.status()

    def last_counts(self):
        """(rows sent to each rank, rows received, bytes stored into peers' buffers) of the last forward."""
        sent = (C.c_uint32 * capi.EP_MAX_WORLD)()
        recv = C.c_uint32()
        nbytes = C.c_uint64()
        self.home._check(self._lib.shrike_ep_last_counts(self._ep, sent, C.byref(recv), C.byref(nbytes)))
        return list(sent[:self.world]), recv.value, nbytes.value

    def _all_to_all(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        if self.world == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out.view(-1), inp.view(-1), group=self.group)

    def forward(self, router: RouterOperands, x: torch.Tensor, y: torch.Tensor,
                hidden: Optional[torch.Tensor] = None) -> None:
        """x: this rank's rows [rows_per_rank, d] in the activation dtype; y in the y dtype."""
        if self._ep is not None:
            ops = router.to_c()
            self.home._check(self._lib.shrike_ep_forward(
                self._ep, _stream(), self.pool._h, C.byref(self.offsets), self.routed.residency_row(0), C.byref(ops),
                C.byref(self.shared) if self.shared is not None else None, _ptr(x), x.shape[0], _ptr(y), _ptr(hidden)))
            return
        cfg, T, G, cap = self.cfg, self.rows, self.world, self.cap
        lib, st = self.home._lib, _stream()
        self.home.encode_router(router, x, self.ids, self.w, self.gate)
        self.home._check(lib.shrike_ep_encode_dispatch(
            self.home._h, st, _ptr(x), _ptr(self.ids), _ptr(self.w), T, G, self.epr, cap, _ptr(self.send_x),
            _ptr(self.send_ids), _ptr(self.send_w), _ptr(self.send_counts), _ptr(self.row_of)))
        self._all_to_all(self.recv_x, self.send_x)
        self._all_to_all(self.recv_ids, self.send_ids)
        self._all_to_all(self.recv_w, self.send_w)
        if cfg.has_shared:
            if T <= capi.MAX_DECODE_TOKENS:
                self.home.encode_decode(self.pool, self.offsets, self.miss_slots, self.w, x, self.y_home, None,
                                        self.shared, self.gate)
            else:
                self.home.encode_prefill(self.pool, self.offsets, self.ids, self.miss_slots, self.w, x, self.y_home,
                                         None, self.shared, self.gate)
        rows = G * cap
        self.routed._check(lib.shrike_ep_encode_local_slots(
            self.routed._h, st, _ptr(self.recv_ids), self.routed.residency_row(0), rows, _ptr(self.slots)))
        rx = self.recv_x.view(rows, cfg.d)
        rw = self.recv_w.view(rows, cfg.top_k)
        rid = self.recv_ids.view(rows, cfg.top_k)
        if rows <= capi.MAX_DECODE_TOKENS:
            self.routed.encode_decode(self.pool, self.offsets, self.slots, rw, rx, self.y_part)
        else:
            self.routed.encode_prefill(self.pool, self.offsets, rid, self.slots, rw, rx, self.y_part)
        self._all_to_all(self.y_back, self.y_part.view(G, cap, cfg.d))
        self.home._check(lib.shrike_ep_encode_combine(
            self.home._h, st, _ptr(self.y_back), _ptr(self.row_of), _ptr(self.y_home), T, G, cap, _ptr(y),
            _ptr(hidden)))

    def routing(self, router: RouterOperands, x: torch.Tensor):
        """(ids, weights) of this rank's rows, through the home handle's router (what forward used)."""
        self.home.encode_router(router, x, self.ids, self.w,
                                torch.zeros(x.shape[0], dtype=torch.float32, device=self.dev) if self.cfg.shared_gated else None)
        return self.ids, self.w

    def exchange_stats(self, router: RouterOperands, x: torch.Tensor, y: torch.Tensor, steps: int) -> dict:
        """What the exchange costs and moves: the layer's time against the same local work with the waits
        already satisfied cannot be separated inside one call, so the two exchange legs are timed as the span
        between the layer's start and its end minus the same rank's one-rank layer (reported by the caller);
        here: counts and bytes of the last forward."""
        self.forward(router, x, y)
        torch.cuda.synchronize()
        if self._ep is None:
            sent = self.send_counts.cpu().tolist()
            row = self.cfg.d * (2 if self.cfg.act_dtype != capi.DTYPE_FP32 else 4)
            return {"rows_sent": sent, "rows_received": None,
                    "bytes_sent": self.world * self.cap * (row + self.cfg.top_k * 8 + self.cfg.d * 4),
                    "exchange": "nccl all_to_all_single, fixed capacity"}
        sent, recv, nbytes = self.last_counts()
        return {"rows_sent": sent, "rows_received": recv, "bytes_sent": nbytes,
                "exchange": "peer stores over NVLink into the destination's buffer (CUDA IPC), only routed rows move"}
