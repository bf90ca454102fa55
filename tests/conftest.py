"""pytest configuration: registers the `gpu` marker and puts the repository
root on sys.path so `oracle` and `dsv4_attn_b200` import without installation."""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
