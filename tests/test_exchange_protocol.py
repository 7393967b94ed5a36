"""The state-exchange kernel's index arithmetic and slot / acknowledgement
protocol, simulated on the CPU for every group size.

tests/csrc/exchange_sim.cpp includes the very header the CUDA kernel uses
(lasp_b200/csrc/exchange_layout.h) and plays all ranks of a group in one
process: every word is written exactly once per step, every element is summed
exactly once with the right decay powers, and the acknowledgements a pusher
waits on are the ones a gatherer writes.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def sim(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("xsim") / "exchange_sim")
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "lasp_b200", "csrc"),
                           os.path.join(ROOT, "tests", "csrc", "exchange_sim.cpp"), "-o", exe])
    return exe


@pytest.mark.parametrize("ranks", [2, 3, 4, 5, 8])
@pytest.mark.parametrize("elems", [1024, 4 * 6 * 16 * 16, 6 * 64 * 48, 2 * 12 * 128 * 128 // 8, 4100])
def test_exchange_protocol_simulation(sim, ranks, elems):
    out = subprocess.run([sim, str(ranks), str(elems), "5"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout + out.stderr
