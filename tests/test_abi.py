"""The shared library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            txt = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"DSX_API\s+[\w\s\*]+?\b(dsx_\w+)\s*\(", txt)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    from deepstrix_b200 import _build
    path = _build.build()
    lib = ctypes.CDLL(path)
    names = _declared()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_host_only_entry_points():
    from deepstrix_b200 import moe
    assert moe.bytes_per_expert(0, 4096, 2048) == 4_456_448     # src/weight_contract.rs:363-366
    assert moe.bytes_per_expert(1, 4096, 2048) == 8_912_896
    assert moe.wi_upper_bound(12, 384, 32) == 12                # het/dispatch.rs:746-748
    assert moe.wi_upper_bound(3072, 384, 32) == 480
    assert moe.wi_upper_bound(3072, 384, 32, 100) == 100
    try:
        moe.bytes_per_expert(7, 4096, 2048)
        assert False
    except moe.DsxError as e:
        assert e.code == -1 and "format" in str(e)


def test_config_byte_model():
    from deepstrix_b200 import CONFIGS
    c = CONFIGS[1]
    assert c.matrix_bytes() == 4_456_448 and c.expert_bytes() == 13_369_344
    assert c.algorithmic_bytes(1, 8) == 124_534_784
    assert abs(c.flops(8192) - 3.728e12) / 3.728e12 < 1e-3
