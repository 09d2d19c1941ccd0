"""The diagnostic gather probe behind ``bench.py --profile gather``."""
import pytest

pytestmark = pytest.mark.gpu


def test_gather_probe_runs_and_reports_a_time():
    """The diagnostic gather probe (bench.py --profile gather) on a small case: all three copy
    methods finish (no bounded wait gives up) and report a positive time."""
    import torch
    from rivoli_b200 import backend as be
    n_rows, n_ctas, n_tiles = 64 * 1024, 8, 4
    pool = torch.ones(n_rows * 576, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(n_rows, dtype=torch.float32, device="cuda")
    rows = torch.randint(0, n_rows, (n_ctas, n_tiles * 128), dtype=torch.int32, device="cuda")
    for method in (0, 1, 2):
        for depth in (1, 2):
            assert be.probe_gather(method, depth, n_ctas, n_tiles, pool, n_rows, scales, rows) > 0.0
