"""The C-ABI library loads on a machine without a GPU and exports every symbol that
``include/dist_moe_b200.h`` declares (no compute call is made here)."""

import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    from dist_moe_b200 import _native

    header = (ROOT / "include" / "dist_moe_b200.h").read_text()
    declared = set(re.findall(r"^\s*(?:int|int64_t)\s+(dm_\w+)\s*\(", header, flags=re.M))
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(_native.lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_native.EXPORTS), declared ^ set(_native.EXPORTS)
    assert _native.lib.dm_version() == 1000


def test_argument_errors_do_not_need_a_gpu():
    from dist_moe_b200 import _native

    assert _native.lib.dm_route_workspace_words(4096, 8, 64) == 2 * 8 * 16 * 8 + 64
    assert _native.lib.dm_publish(None, None, 0, None, None, 0, 0, 0, 0, 0, None, None) == -1
    assert _native.lib.dm_quant_mxfp8_row(None, None, 1, 32, None, 0, None, 0, 0, None) == -1


def test_product_package_does_not_import_the_oracle():
    for path in (ROOT / "dist_moe_b200").rglob("*.py"):
        text = path.read_text()
        assert "import oracle" not in text and "from oracle" not in text, path
