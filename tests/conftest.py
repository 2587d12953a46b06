import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (ROOT, os.path.join(ROOT, "ascend-moe-engine_b200"), os.path.join(ROOT, "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """Attention tolerance outcomes of the run: which comparisons also met the per-element bound."""
    try:
        import scenarios
    except Exception:  # pragma: no cover
        return
    records = scenarios.TOLERANCE_RECORDS
    if not records:
        return
    held = sum(1 for r in records if r["element_bound_excess"] <= 0.0)
    terminalreporter.write_line(f"attention comparisons: {len(records)}; per-element bound 2e-3 + 1e-2*|ref| held in {held}")
    for r in records:
        if r["element_bound_excess"] > 0.0:
            terminalreporter.write_line(
                f"  per-element bound exceeded by {r['element_bound_excess']:.3e} (row bound margin "
                f"{-r['row_bound_excess']:.3e}, max |ref| {r['max_abs_ref']:.3g}): {r['what']}")
    path = os.environ.get("B200KV_TOLERANCE_REPORT")
    if path:
        import json

        with open(path, "w") as f:
            json.dump(records, f, indent=1)
