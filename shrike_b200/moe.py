"""Host-side mirror of the reference's MoE dispatch surface over the C ABI.

Class and method names follow the Swift wrappers they stand for
(sources/Shrike/Kernels/MoE/MoE.swift, sources/Shrike/Kernels/Prefill/MoE,
sources/Shrike/Infrastructure/Streaming/ExpertCellArena.swift); arguments keep
their meaning. Device memory and streams come from torch; nothing here
computes: every method validates and forwards to libshrike_b200.so and raises
`ShrikeError` with the library's message on a non-zero return.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import capi


class ShrikeError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"shrike_b200 error {code}: {message}")
        self.code = code


_TORCH_ACT = {capi.DTYPE_BF16: torch.bfloat16, capi.DTYPE_FP16: torch.float16, capi.DTYPE_FP32: torch.float32}


@dataclass
class MoEConfig:
    """Arguments of `MoE.init` (MoE.swift:94-106) plus the dtypes."""
    d: int
    f: int
    num_experts: int
    top_k: int
    weight_bits: int = 4
    group_size: int = 64
    meta_dtype: int = capi.DTYPE_BF16
    act_dtype: int = capi.DTYPE_BF16
    activation: int = capi.ACT_SILU
    expert_bias: bool = False
    router_kind: int = capi.ROUTER_SOFTMAX
    routed_scaling: float = 1.0
    router_weight_bits: int = 0
    round_route_weights_f16: bool = True
    has_shared: bool = False
    shared_gated: bool = False
    shared_f: int = 0
    max_tokens: int = 16
    y_dtype: Optional[int] = None   # dtype of y; None = the activation dtype

    @property
    def out_dtype(self) -> int:
        return self.act_dtype if self.y_dtype is None else self.y_dtype

    def to_c(self) -> capi.MoEConfig:
        return capi.MoEConfig(
            self.d, self.f, self.num_experts, self.top_k, self.weight_bits, self.group_size,
            self.meta_dtype, self.act_dtype, self.activation, int(self.expert_bias), self.router_kind,
            float(self.routed_scaling), self.router_weight_bits, int(self.round_route_weights_f16),
            int(self.has_shared), int(self.shared_gated), self.shared_f if self.has_shared else 0,
            self.max_tokens, self.out_dtype)

    @property
    def torch_act_dtype(self) -> torch.dtype:
        return _TORCH_ACT[self.act_dtype]

    @property
    def torch_y_dtype(self) -> torch.dtype:
        return _TORCH_ACT[self.out_dtype]


def expert_offsets(config: MoEConfig, shared: bool = False) -> tuple[capi.ExpertOffsets, int]:
    """`CPUExpertFFN.Offsets` / `Model.routedExpertOffsets`: offsets and block size in bytes."""
    lib = capi.load()
    off = capi.ExpertOffsets()
    size = C.c_uint64()
    cfg = config.to_c()
    rc = lib.shrike_expert_offsets_make(C.byref(cfg), int(shared), C.byref(off), C.byref(size))
    if rc:
        raise ShrikeError(rc, lib.shrike_last_error(None).decode())
    return off, size.value


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("device operands must be contiguous CUDA tensors")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


@dataclass
class RouterOperands:
    """Buffers of `MoE.encodeRouter` (MoE.swift:249-261); bf16 vectors as int16/bfloat16 tensors."""
    weights: torch.Tensor
    scales: Optional[torch.Tensor] = None
    biases: Optional[torch.Tensor] = None
    effective_scale: Optional[torch.Tensor] = None
    per_expert_scale: Optional[torch.Tensor] = None
    logit_bias: Optional[torch.Tensor] = None
    shared_gate: Optional[torch.Tensor] = None

    def to_c(self) -> capi.RouterOperands:
        return capi.RouterOperands(_ptr(self.weights), _ptr(self.scales), _ptr(self.biases),
                                   _ptr(self.effective_scale), _ptr(self.per_expert_scale),
                                   _ptr(self.logit_bias), _ptr(self.shared_gate))


class MoE:
    """Stands for `final class MoE` and the prefill MoE wrappers; owns the workspace."""

    def __init__(self, config: MoEConfig, device: int = 0):
        self._lib = capi.load()
        self.config = config
        self.device = device
        handle = C.c_void_p()
        cfg = config.to_c()
        rc = self._lib.shrike_moe_create(C.byref(cfg), device, C.byref(handle))
        if rc:
            raise ShrikeError(rc, self._lib.shrike_last_error(None).decode())
        self._h = handle
        self._residency_ptr = None
        self._residency_layers = 0

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.shrike_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int) -> None:
        if rc:
            raise ShrikeError(rc, self._lib.shrike_last_error(self._h).decode())

    def status(self) -> None:
        """Synchronises the current stream and raises if a kernel reported a failure."""
        self._check(self._lib.shrike_moe_status(self._h, _stream()))

    # -- residency table (ExpertResidencyTable.swift:4-19) ---------------------
    def create_residency(self, layers: int) -> None:
        p = C.c_void_p()
        self._check(self._lib.shrike_residency_create(self._h, layers, C.byref(p)))
        self._residency_ptr = p.value
        self._residency_layers = layers

    def residency_row(self, layer: int) -> int:
        if self._residency_ptr is None or layer >= self._residency_layers:
            raise ValueError("residency table not created for this layer")
        return self._residency_ptr + layer * self.config.num_experts * 8

    def residency_set(self, layer: int, expert: int, slot: int, state: int) -> None:
        self._check(self._lib.shrike_residency_set(self._h, layer, expert, slot, state, _stream()))

    def residency_set_layer_identity(self, layer: int, first_cell: int) -> None:
        self._check(self._lib.shrike_residency_set_layer_identity(self._h, layer, first_cell, _stream()))

    # -- the path ------------------------------------------------------------
    def encode_router(self, operands: RouterOperands, hidden: torch.Tensor, out_indices: torch.Tensor,
                      out_weights: torch.Tensor, out_shared_gate: Optional[torch.Tensor] = None,
                      query_count: Optional[int] = None, hidden_stride_elements: Optional[int] = None) -> None:
        """`MoE.encodeRouter` / `PrefillRouter.encodeBlock`."""
        q = hidden.shape[0] if query_count is None else query_count
        stride = hidden.stride(0) if hidden_stride_elements is None else hidden_stride_elements
        ops = operands.to_c()
        if not hidden.is_cuda:
            raise ValueError("hidden must be a CUDA tensor")
        self._check(self._lib.shrike_encode_router(self._h, _stream(), C.byref(ops), hidden.data_ptr(), q, stride,
                                                   _ptr(out_indices), _ptr(out_weights), _ptr(out_shared_gate)))

    def encode_residency_classification(self, topk_indices: torch.Tensor, layer: int, resolved_slots: torch.Tensor,
                                        counts: Optional[torch.Tensor] = None,
                                        miss_positions: Optional[torch.Tensor] = None,
                                        miss_experts: Optional[torch.Tensor] = None,
                                        query_count: Optional[int] = None) -> None:
        """`MoE.encodeResidencyClassification`."""
        q = topk_indices.shape[0] if query_count is None else query_count
        self._check(self._lib.shrike_encode_residency_classification(
            self._h, _stream(), _ptr(topk_indices), self.residency_row(layer), q, _ptr(resolved_slots),
            _ptr(counts), _ptr(miss_positions), _ptr(miss_experts)))

    def encode_decode(self, pool: "ExpertCellArena", routed_offsets: capi.ExpertOffsets,
                      resolved_slots: torch.Tensor, routing_weights: torch.Tensor, x: torch.Tensor,
                      y: torch.Tensor, hidden: Optional[torch.Tensor] = None,
                      shared: Optional[capi.SharedExpert] = None, shared_gate: Optional[torch.Tensor] = None,
                      io_status: Optional[torch.Tensor] = None, query_count: Optional[int] = None) -> None:
        """encodeSharedExpertWork + `MoE.encodeSpecPhase1U16Load` + `MoE.encodeSpecPhase2Reduce`."""
        q = x.shape[0] if query_count is None else query_count
        self._check(self._lib.shrike_encode_moe_decode(
            self._h, _stream(), pool._h, C.byref(routed_offsets), _ptr(resolved_slots), _ptr(routing_weights),
            _ptr(x), q, C.byref(shared) if shared is not None else None, _ptr(shared_gate), _ptr(io_status),
            _ptr(y), _ptr(hidden)))

    def encode_decode_plan(self, pool: "ExpertCellArena", resolved_slots: torch.Tensor, x: torch.Tensor,
                           io_status: Optional[torch.Tensor] = None, query_count: Optional[int] = None) -> None:
        q = x.shape[0] if query_count is None else query_count
        self._check(self._lib.shrike_encode_decode_plan(self._h, _stream(), pool._h, _ptr(resolved_slots), _ptr(x),
                                                        q, _ptr(io_status)))

    def encode_phase1(self, pool: "ExpertCellArena", routed_offsets: capi.ExpertOffsets, query_count: int,
                      shared: Optional[capi.SharedExpert] = None) -> None:
        """`MoE.encodeSpecPhase1U16Load` (+ the shared expert's gate/up grid)."""
        self._check(self._lib.shrike_encode_phase1(self._h, _stream(), pool._h, C.byref(routed_offsets),
                                                   C.byref(shared) if shared is not None else None, query_count))

    def encode_phase2_reduce(self, pool: "ExpertCellArena", routed_offsets: capi.ExpertOffsets,
                             routing_weights: torch.Tensor, y: torch.Tensor, query_count: int,
                             hidden: Optional[torch.Tensor] = None, shared: Optional[capi.SharedExpert] = None,
                             shared_gate: Optional[torch.Tensor] = None) -> None:
        """`MoE.encodeSpecPhase2Reduce` (+ the shared expert's down projection)."""
        self._check(self._lib.shrike_encode_phase2_reduce(
            self._h, _stream(), pool._h, C.byref(routed_offsets), _ptr(routing_weights),
            C.byref(shared) if shared is not None else None, _ptr(shared_gate), query_count, _ptr(y), _ptr(hidden)))

    def encode_route_decode(self, operands: RouterOperands, layer: int, pool: "ExpertCellArena",
                            hidden: torch.Tensor, out_indices: torch.Tensor, out_weights: torch.Tensor,
                            out_shared_gate: Optional[torch.Tensor] = None,
                            out_resolved_slots: Optional[torch.Tensor] = None,
                            out_counts: Optional[torch.Tensor] = None, io_status: Optional[torch.Tensor] = None,
                            query_count: Optional[int] = None, hidden_stride_elements: Optional[int] = None) -> None:
        """Router + residency classification + decode work lists in one launch."""
        q = hidden.shape[0] if query_count is None else query_count
        stride = hidden.stride(0) if hidden_stride_elements is None else hidden_stride_elements
        ops = operands.to_c()
        self._check(self._lib.shrike_encode_route_decode(
            self._h, _stream(), C.byref(ops), self.residency_row(layer), pool._h, hidden.data_ptr(), q, stride,
            _ptr(io_status), _ptr(out_indices), _ptr(out_weights), _ptr(out_shared_gate),
            _ptr(out_resolved_slots), _ptr(out_counts)))

    def encode_decode_layer(self, pool: "ExpertCellArena", routed_offsets: capi.ExpertOffsets, layer: int,
                            router: RouterOperands, x: torch.Tensor, y: torch.Tensor,
                            hidden: Optional[torch.Tensor] = None, shared: Optional[capi.SharedExpert] = None,
                            out_indices: Optional[torch.Tensor] = None, out_weights: Optional[torch.Tensor] = None,
                            io_status: Optional[torch.Tensor] = None, query_count: Optional[int] = None) -> None:
        """One decode layer (route -> phase 1 -> phase 2) as three dependent launches."""
        q = x.shape[0] if query_count is None else query_count
        ops = router.to_c()
        self._check(self._lib.shrike_encode_decode_layer(
            self._h, _stream(), pool._h, C.byref(routed_offsets), self.residency_row(layer), C.byref(ops),
            C.byref(shared) if shared is not None else None, _ptr(x), q, _ptr(io_status), _ptr(out_indices),
            _ptr(out_weights), _ptr(y), _ptr(hidden)))

    def encode_prefill(self, pool: "ExpertCellArena", routed_offsets: capi.ExpertOffsets,
                       topk_indices: torch.Tensor, resolved_slots: torch.Tensor, routing_weights: torch.Tensor,
                       x: torch.Tensor, y: torch.Tensor, hidden: Optional[torch.Tensor] = None,
                       shared: Optional[capi.SharedExpert] = None, shared_gate: Optional[torch.Tensor] = None,
                       query_count: Optional[int] = None) -> None:
        """buildPrefillRoutes + encodeGroupedExpertGEMMs + shared chunk + encodeReduceTokenMajor + residual adds."""
        q = x.shape[0] if query_count is None else query_count
        self._check(self._lib.shrike_encode_moe_prefill(
            self._h, _stream(), pool._h, C.byref(routed_offsets), _ptr(topk_indices), _ptr(resolved_slots),
            _ptr(routing_weights), _ptr(x), q, C.byref(shared) if shared is not None else None,
            _ptr(shared_gate), _ptr(y), _ptr(hidden)))

    def group_token_expert_pairs(self, topk_indices: torch.Tensor, routing_weights: Optional[torch.Tensor],
                                 sorted_pairs: torch.Tensor, per_expert_offsets: torch.Tensor,
                                 per_expert_counts: torch.Tensor, query_count: Optional[int] = None) -> None:
        """`PrefillMoEGrouping.groupTokenExpertPairs` on the device."""
        q = topk_indices.shape[0] if query_count is None else query_count
        self._check(self._lib.shrike_encode_group_pairs(
            self._h, _stream(), _ptr(topk_indices), _ptr(routing_weights), q, _ptr(sorted_pairs),
            _ptr(per_expert_offsets), _ptr(per_expert_counts)))

    def layer_forward_host(self, pool: "ExpertCellArena", routed_offsets: capi.ExpertOffsets, layer: int,
                           router: RouterOperands, x_host: torch.Tensor, y_host: torch.Tensor,
                           shared: Optional[capi.SharedExpert] = None, ids_host: Optional[torch.Tensor] = None,
                           weights_host: Optional[torch.Tensor] = None) -> None:
        """One layer with host activations in and out (copies inside the call)."""
        for t in (x_host, y_host, ids_host, weights_host):
            if t is not None and (t.is_cuda or not t.is_contiguous()):
                raise ValueError("host operands must be contiguous CPU tensors")
        ops = router.to_c()
        self._check(self._lib.shrike_moe_layer_forward_host(
            self._h, _stream(), pool._h, C.byref(routed_offsets), self.residency_row(layer), C.byref(ops),
            C.byref(shared) if shared is not None else None, x_host.data_ptr(), x_host.shape[0],
            y_host.data_ptr(), ids_host.data_ptr() if ids_host is not None else None,
            weights_host.data_ptr() if weights_host is not None else None))


class DecodeStack:
    """Stacked MoE layers behind `shrike_decode_stack_forward_host`: one decode step with host activations in
    and out (copies inside the call). `layers`: (moe, pool, routed_offsets, layer index, router, shared)."""

    def __init__(self, layers, max_rows: int):
        self._lib = capi.load()
        self._keep = []
        arr = (capi.StackLayer * len(layers))()
        for i, (moe, pool, off, layer, router, shared) in enumerate(layers):
            ops = router.to_c()
            self._keep += [ops, off, shared, router]
            arr[i] = capi.StackLayer(moe._h, pool._h, C.pointer(off), moe.residency_row(layer), C.pointer(ops),
                                     C.pointer(shared) if shared is not None else None)
        self._first = layers[0][0]
        h = C.c_void_p()
        self._first._check(self._lib.shrike_decode_stack_create(arr, len(layers), max_rows, C.byref(h)))
        self._h = h

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.shrike_decode_stack_destroy(self._h)
            self._h = None

    def forward_host(self, rows_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """rows_host [(layers + 1), T, d]: block 0 enters layer 0, block l is added to the residual stream
        before layer l; out_host [T, d] receives the stream after the last layer."""
        for t in (rows_host, out_host):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("host operands must be contiguous CPU tensors")
        self._first._check(self._lib.shrike_decode_stack_forward_host(
            self._h, _stream(), rows_host.data_ptr(), rows_host.shape[1], out_host.data_ptr()))


def encode_router_static(config: MoEConfig, operands: RouterOperands, hidden: torch.Tensor,
                         out_indices: torch.Tensor, out_weights: torch.Tensor,
                         out_shared_gate: Optional[torch.Tensor] = None, query_count: Optional[int] = None,
                         hidden_stride_elements: Optional[int] = None) -> None:
    """The router without a handle and without any allocation (`shrike_encode_router_static`).

    For hosts that cannot call cudaMalloc once their expert pool owns the device's memory or inside
    their decode loop: the logits scratch is a 64 KiB array built into the library, so at most 64 rows
    and 256 experts per call. Calls that overlap on the GPU share that array and race; make the first
    call on a device outside stream capture.
    """
    lib = capi.load()
    q = hidden.shape[0] if query_count is None else query_count
    stride = hidden.stride(0) if hidden_stride_elements is None else hidden_stride_elements
    cfg = config.to_c()
    ops = operands.to_c()
    text = C.create_string_buffer(256)
    rc = lib.shrike_encode_router_static(C.byref(cfg), _stream(), C.byref(ops), hidden.data_ptr(), q, stride,
                                         _ptr(out_indices), _ptr(out_weights), _ptr(out_shared_gate), text, 256)
    if rc:
        raise ShrikeError(rc, text.value.decode())


class ExpertCellArena:
    """`ExpertCellArena` (ExpertCellArena.swift:16-132): cells of whole expert blocks in HBM."""

    def __init__(self, moe: MoE, cells: int, cell_stride: int, chunks: int = 1):
        self._moe = moe
        self._lib = moe._lib
        self.cells = cells
        self.cell_stride = cell_stride
        h = C.c_void_p()
        moe._check(self._lib.shrike_pool_create(moe._h, cells, cell_stride, chunks, C.byref(h)))
        self._h = h

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.shrike_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def upload(self, cell: int, block) -> None:
        """Copies one packed expert block (bytes / numpy uint8 array) into a cell."""
        import numpy as np
        buf = np.ascontiguousarray(np.frombuffer(block, dtype=np.uint8) if isinstance(block, (bytes, bytearray)) else block)
        self._moe._check(self._lib.shrike_pool_upload(self._h, cell, buf.ctypes.data, buf.nbytes, _stream()))
        torch.cuda.current_stream().synchronize()  # the host buffer may go away after return

    def download(self, cell: int, nbytes: int):
        import numpy as np
        out = np.empty(nbytes, dtype=np.uint8)
        self._moe._check(self._lib.shrike_pool_download(self._h, cell, out.ctypes.data, nbytes, _stream()))
        return out

    def cell_address(self, cell: int) -> int:
        p = C.c_void_p()
        self._moe._check(self._lib.shrike_pool_cell_address(self._h, cell, C.byref(p)))
        return p.value

    def fill_synthetic(self, first_cell: int, count: int, seed: int, layer: int, first_expert: int = 0,
                       shared: bool = False) -> None:
        self._moe._check(self._lib.shrike_pool_fill_synthetic(
            self._moe._h, self._h, first_cell, count, seed, layer, first_expert, int(shared), _stream()))


def round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m
