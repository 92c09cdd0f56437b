"""Shared pytest configuration: the `gpu` marker, import paths and golden fixtures."""

import sys
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
GOLDEN = REPO / "tests" / "golden"
for path in (str(REPO), str(GOLDEN)):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_ops():
    """Per-operator outputs of the reference: ops.pt (fp32, bf16) and ops_fp16.pt."""
    return {**torch.load(GOLDEN / "ops.pt", weights_only=False),
            **torch.load(GOLDEN / "ops_fp16.pt", weights_only=False)}


@pytest.fixture(scope="session")
def golden_tiny():
    return {tag: torch.load(GOLDEN / f"qwen2_tiny_{tag}.pt", weights_only=False)
            for tag in ("fp32", "bf16", "fp16")}
