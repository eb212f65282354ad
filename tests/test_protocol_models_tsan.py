"""The peer-memory protocols restated with std::atomic (same memory orders as the kernels), one thread per rank,
run under ThreadSanitizer on the host: the correct orders are race free, two deliberately broken configurations
are caught."""
import os
import shutil
import subprocess

import pytest

SRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ulacache_b200", "csrc", "models",
                   "protocol_model.cpp")


@pytest.fixture(scope="module")
def model_binary(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    out = str(tmp_path_factory.mktemp("tsan") / "protocol_model")
    res = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-pthread", SRC, "-o", out],
                         capture_output=True, text=True)
    if res.returncode != 0:
        pytest.skip("ThreadSanitizer runtime not available: " + res.stderr[-300:])
    return out


def _run(binary, *args):
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66")
    return subprocess.run([binary, *args], capture_output=True, text=True, timeout=300, env=env)


@pytest.mark.parametrize("scenario,ranks", [("barrier", 4), ("barrier", 8), ("lifetime", 4), ("tagged", 4), ("tagged", 8)])
def test_protocols_are_race_free_under_tsan(model_binary, scenario, ranks):
    res = _run(model_binary, scenario, str(ranks), "120")
    assert res.returncode == 0, res.stdout[-500:] + res.stderr[-1500:]
    assert "ThreadSanitizer" not in res.stderr and res.stdout.strip().endswith("ok")


def test_broken_configurations_are_caught(model_binary):
    one_slot = _run(model_binary, "tagged-one-slot")            # a sender laps a slow reader: its wait runs out
    assert one_slot.returncode == 3 and "timeout" in one_slot.stdout
    relaxed = _run(model_binary, "barrier-relaxed", "4", "50")  # flags without release order: a payload race
    assert relaxed.returncode == 66 and "data race" in relaxed.stderr
