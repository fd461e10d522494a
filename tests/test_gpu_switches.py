"""Every IERT_* switch set to 0, one at a time, each in a process of its own (the switches are
read from the environment when the libraries load), on the workload of tests/switch_probe.py,
against the same workload with every switch at its default.

Where the switch changes who does the work but not the arithmetic (ordinary launches instead
of programmatic dependent ones; the last split of a tile adding alone; the residual read and
written by the epilogue instead of added by TMA; another order of the tiles) the results are
equal to the bit; where it changes the order of a sum or the kernel (no parts in the last wave,
the mma.sync prompt attention, cp.async pages, a separate rotation kernel, an even cut of the
keys, split-K projections in one-token steps, norms as kernels of their own) they agree within
the bfloat16 tolerance of the logits.
"""
import os
import subprocess
import sys

import pytest
import torch

from helpers import compare

pytestmark = pytest.mark.gpu
TESTS = os.path.dirname(os.path.abspath(__file__))

SWITCHES = {            # switch -> are the results equal to the bit with it off?
    "IERT_PDL": True,
    "IERT_GEMM_COOP": True,
    "IERT_GEMM_TMA_OUT": True,
    "IERT_GEMM_TILE_GROUPS": True,
    "IERT_GEMM_TAIL_PARTS": False,
    "IERT_ATTN_TC": False,
    "IERT_FUSED_ROPE": False,
    "IERT_DECODE_TMA": False,
    "IERT_DECODE_BALANCE": False,
    "IERT_GEMM_ROWS_MAX": False,        # 0: one-token projections on the tcgen05 kernel with split-K
    "IERT_NORM_AHEAD": False,           # 0: every norm a kernel of its own
}


@pytest.fixture(scope="module")
def runs(tmp_path_factory):
    """All the processes at once (each holds a two-layer model: they share the device easily)."""
    root = tmp_path_factory.mktemp("switches")
    procs = {}
    for name in [None] + list(SWITCHES):
        env = {k: v for k, v in os.environ.items() if not (k.startswith("IERT_") and k in SWITCHES)}
        if name:
            env[name] = "0"
        path = str(root / f"{name or 'default'}.pt")
        procs[name] = (path, subprocess.Popen([sys.executable, os.path.join(TESTS, "switch_probe.py"), path], env=env,
                                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    out = {}
    for name, (path, proc) in procs.items():
        log, _ = proc.communicate(timeout=900)
        out[name] = (proc.returncode, log, path)
    return out


def load(runs, name):
    rc, log, path = runs[name]
    assert rc == 0, f"{name or 'default'}: the probe failed\n{log[-3000:]}"
    return torch.load(path)


@pytest.mark.parametrize("switch", list(SWITCHES))
def test_switch_off_changes_no_result(runs, switch):
    want, got = load(runs, None), load(runs, switch)
    assert set(want) == set(got)
    for key, ref in want.items():
        if key.endswith("_err"):
            # the projection alone against the float64 product: 2e-3 * sqrt(K) / 2, as in its own tests
            assert got[key] <= 2e-3 * (14336 ** 0.5) * 0.5, f"{switch}=0: {key} = {got[key]}"
            continue
        if SWITCHES[switch]:
            assert torch.equal(got[key], ref), f"{switch}=0: {key} differs from the default run"
        elif key.startswith("gemm_"):
            assert torch.allclose(got[key], ref, atol=2e-3 * (14336 ** 0.5) * 0.5, rtol=0), f"{switch}=0: {key}"
        else:
            compare(got[key], ref, "bfloat16", f"{switch}=0: {key}")


def test_the_default_run_is_repeatable(runs):
    """Two processes with the same switches give the same bits (IERT_PDL=0 changes only how kernels
    are launched, so it doubles as the second run)."""
    a, b = load(runs, None), load(runs, "IERT_PDL")
    for key in a:
        if not key.endswith("_err"):
            assert torch.equal(a[key], b[key]), key
