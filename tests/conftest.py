import json
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name: str):
    return torch.load(GOLDEN / name, map_location="cpu")


def same_host_as_golden() -> bool:
    """bf16 matmuls on the CPU round differently across CPU generations, so golden
    files are bit-reproducible only on the kind of host that wrote them."""
    recorded = json.loads((GOLDEN / "HOST.json").read_text())
    model, flags = "", ""
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name") and not model:
                model = line.split(":", 1)[1].strip()
            if line.startswith("flags") and not flags:
                names = line.split(":", 1)[1].split()
                flags = " ".join(sorted(n for n in names if n.startswith(("avx", "amx"))))
    except OSError:
        return False
    return (model == recorded["cpu_model"] and flags == recorded["simd_flags"]
            and torch.__version__ == recorded["torch"])


# North-star tolerance for floating-point parity (bf16 storage, fp32 accumulation).
ATOL, RTOL = 2e-2, 1e-2


def assert_parity(actual: torch.Tensor, expected: torch.Tensor, what: str, exact: bool = False):
    actual, expected = actual.detach().cpu(), expected.detach().cpu()
    assert actual.shape == expected.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}"
    if exact:
        assert torch.equal(actual, expected), (
            f"{what}: not bit-identical; max abs diff "
            f"{(actual.float() - expected.float()).abs().max().item():.4g}")
        return
    diff = (actual.float() - expected.float()).abs()
    bound = ATOL + RTOL * expected.float().abs()
    worst = (diff - bound).max().item()
    assert worst <= 0, f"{what}: max abs diff {diff.max().item():.4g} exceeds {ATOL} + {RTOL}*|ref| by {worst:.4g}"


@pytest.fixture(scope="session")
def exact_cpu() -> bool:
    return same_host_as_golden()
