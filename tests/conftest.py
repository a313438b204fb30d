import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The achieved errors of the comparisons that ran: the worst of each kind, beside its bound."""
    import json

    import helpers
    if not helpers.ACHIEVED:
        return
    worst = {}
    for row in helpers.ACHIEVED:
        best = worst.get(row["kind"])
        if best is None or row["error"] > best["error"]:
            worst[row["kind"]] = row
    terminalreporter.write_sep("-", "achieved errors (worst of each kind)")
    for kind in sorted(worst):
        row = worst[kind]
        terminalreporter.write_line(f"{kind}: {row['error']:.3e} (bound {row['bound']:.1e}) at {row['what']}")
    path = os.environ.get("LLMPLAYER_B200_ERROR_LOG")
    if path:
        with open(path, "w") as fh:
            json.dump(helpers.ACHIEVED, fh)
