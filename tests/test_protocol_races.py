"""Race tests of the peer-memory flag protocols on the CPU.

``tests/native/ep_exchange_race.cc`` does the same for the expert-parallel token exchange (``parallel/nvlink_ep.py``,
``csrc/ep.cu``): counts published into peers' tables, slots derived from the table, rows pushed into the owners' receive
buffers, arrival counters, and the way back; the negative control copies a receive buffer out without waiting for its
arrival counter.

``tests/native/fsdp_flags_race.cc`` runs the version-flag state machine of the NVLink FSDP transport
(``parallel/nvlink_comm.py``, ``csrc/comm.cu``) with two threads per rank (compute stream, reduce stream) on plain
arrays, using the same flag primitives as the kernels (``csrc/protocol.h`` built for the host). Under ThreadSanitizer
the protocol as shipped must be free of data races, and the build that leaves out the staging-buffer guard
(``NvlinkComm.before_grad_writes``) must be reported, which shows that the harness sees the hazard the guard exists for.
"""

import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "native", "fsdp_flags_race.cc")
SRC_EP = os.path.join(HERE, "native", "ep_exchange_race.cc")
INC = os.path.join(os.path.dirname(HERE), "torchtitan_b200", "csrc")


def _build(tmp_path, name, extra=(), src=SRC):
    exe = str(tmp_path / name)
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-pthread", "-I", INC, *extra, src, "-o", exe]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        pytest.skip(f"ThreadSanitizer build not available here: {res.stderr[-300:]}")
    return exe


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_fsdp_flag_protocol_has_no_data_race_and_the_guard_is_needed(tmp_path):
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66")
    good = subprocess.run([_build(tmp_path, "good")], capture_output=True, text=True, env=env, timeout=600)
    assert good.returncode == 0, good.stderr[-2000:]
    assert "ThreadSanitizer" not in good.stderr and "checksum" in good.stdout
    bad_exe = _build(tmp_path, "bad", ["-DDROP_STAGING_WAIT"])
    seen = False
    for _ in range(3):                               # the report needs both accesses in the detector's window
        bad = subprocess.run([bad_exe], capture_output=True, text=True, env=env, timeout=600)
        if "ThreadSanitizer: data race" in bad.stderr:
            seen = True
            break
    assert seen, "the build without the staging-buffer guard was not reported"
    assert "staging" in bad.stderr or "reduce_stream" in bad.stderr or "compute_stream" in bad.stderr


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_expert_exchange_protocol_has_no_data_race(tmp_path):
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66")
    for name, flags in (("double", []), ("single", ["-DSINGLE_BUFFER"])):
        good = subprocess.run([_build(tmp_path, name, flags, SRC_EP)], capture_output=True, text=True, env=env, timeout=600)
        assert good.returncode == 0, (name, good.stdout, good.stderr[-2000:])      # 0 also means every row came back
        assert "ThreadSanitizer" not in good.stderr
    bad_exe = _build(tmp_path, "nowait", ["-DDROP_ARRIVE_WAIT"], SRC_EP)
    reports = [subprocess.run([bad_exe], capture_output=True, text=True, env=env, timeout=600).stderr for _ in range(3)]
    assert any("ThreadSanitizer: data race" in r for r in reports), "copying out before the arrivals was not reported"
