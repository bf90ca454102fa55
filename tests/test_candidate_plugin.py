"""The harness plug-in obeys the reference's discovery contract: literal
top-level NAME / VARIANT assignments found by regular expression over the file
text (bench/bench/candidates/__init__.py:18-46), and a `candidate` callable."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
NAME_RE = re.compile(r"""^\s*NAME\s*=\s*["']([^"']+)["']""", re.MULTILINE)
VARIANT_RE = re.compile(r"""^\s*VARIANT\s*=\s*["']([^"']+)["']""", re.MULTILINE)


def test_plugin_is_discoverable_by_source_regex():
    text = (ROOT / "dsv4_attn_b200" / "candidates" / "hca_b200_decode.py").read_text()
    assert NAME_RE.search(text).group(1) == "hca_b200_decode"
    assert VARIANT_RE.search(text).group(1) == "hca_decode"
    assert re.search(r"^def candidate\(inputs, \*, spec\)", text, re.MULTILINE)


def test_plugin_binds_the_exported_symbol():
    import importlib
    mod = importlib.import_module("dsv4_attn_b200.candidates.hca_b200_decode")
    fn = mod._load()
    assert fn.restype is not None and len(fn.argtypes) == 19
