import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (HERE, ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_terminal_summary(terminalreporter):
    """The worst errors the bfloat16 comparisons saw, beside their bounds (``gpu_util.observe``)."""
    try:
        import gpu_util
    except Exception:
        return
    if not gpu_util.OBSERVED:
        return
    terminalreporter.write_sep("-", "observed errors (fraction of the largest |logit|; bound)")
    for what, (frac, bound) in sorted(gpu_util.OBSERVED.items()):
        terminalreporter.write_line(f"{what}: {frac:.5f}  (bound {bound:.5f})")
    path = os.environ.get("ZLLM_OBSERVED_FILE")
    if path:
        import json
        with open(path, "w") as f:
            json.dump({k: list(v) for k, v in gpu_util.OBSERVED.items()}, f, indent=1)
