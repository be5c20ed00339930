"""The C-ABI library loads and exports every symbol the header declares (no compute, no GPU)."""
import ctypes
import re
from pathlib import Path

from shrike_b200 import build, capi

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "shrike_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(shrike_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    build.build()
    names = declared_symbols()
    assert len(names) >= 15
    lib = ctypes.CDLL(str(capi.LIB_PATH))
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(capi.SIGNATURES) == names, "capi.py and the header disagree"


def test_offsets_entry_point_needs_no_gpu():
    import fixtures as fx
    from shrike_b200.moe import expert_offsets
    off, size = expert_offsets(fx.qwen_config())
    assert size == 1_769_472 and off.gate_s == 524_288 and off.up_w == 589_824 and off.down_w == 1_179_648
    off, size = expert_offsets(fx.gpt_oss_config(group_size=32))
    assert size == 15_569_280 and off.gate_ab % 16 == 0
    off, size = expert_offsets(fx.kimi_config())
    assert size == 7_520_256


def test_create_fails_loudly_without_a_device():
    import pytest
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    import fixtures as fx
    from shrike_b200.moe import MoE, ShrikeError
    with pytest.raises(ShrikeError) as e:
        MoE(fx.qwen_config())
    assert "no CUDA device" in str(e.value)


def test_misaligned_router_operands_are_refused_before_any_launch():
    """The router kernels use 16-byte loads on the weight rows and 8/16-byte loads on the activations; an
    offset pointer comes back as SHRIKE_EINVAL from the argument checks (no device is touched: this runs
    without a GPU), never as a misaligned-address fault."""
    import ctypes as C
    import fixtures as fx
    lib = capi.load()
    cfg = fx.qwen_config(act_dtype=capi.DTYPE_FP32, shared_gated=False).to_c()
    text = C.create_string_buffer(256)
    base = 0x7f0000000000   # never dereferenced: the checks come first

    def call(weights, hidden, eff=None):
        ops = capi.RouterOperands(weights, None, None, eff, None, None, None)
        return lib.shrike_encode_router_static(C.byref(cfg), None, C.byref(ops), hidden, 1, 2048, base, base, None,
                                               text, 256)

    assert call(base + 4, base) == capi.EINVAL and b"16-byte" in text.value
    assert call(base, base + 8) == capi.EINVAL and b"hidden" in text.value
    assert call(base, base, base + 2) == capi.EINVAL and b"effective_scale" in text.value
    cfg16 = fx.qwen_config(shared_gated=False).to_c()   # bf16 activations: 8 bytes suffice, 4 do not
    ops = capi.RouterOperands(base, None, None, None, None, None, None)
    assert lib.shrike_encode_router_static(C.byref(cfg16), None, C.byref(ops), base + 4, 1, 2048, base, base, None,
                                           text, 256) == capi.EINVAL
