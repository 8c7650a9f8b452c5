"""pytest configuration: registers the `gpu` marker and puts the package
directory (which holds tk_evo_attention_layer.py, as in the reference's
evo_h100/) and the repository root (oracle/) on sys.path."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "megakernel-exploration_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
