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
    from shrike_b200 import fixtures as fx
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
    from shrike_b200 import fixtures as fx
    from shrike_b200.moe import MoE, ShrikeError
    with pytest.raises(ShrikeError) as e:
        MoE(fx.qwen_config())
    assert "no CUDA device" in str(e.value)
