"""CPU suite, world_size 2 over gloo: the expert-parallel exchange reproduces the single-device block.
Checked against the golden output generated from the reference (tests/golden/moe.npz, case "small")."""
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

HERE = Path(__file__).resolve().parent


def _wait_all(procs, timeout):
    """Wait for every rank; as soon as one fails or the time runs out, the others are killed, so that no rank is
    left inside a collective holding a device."""
    import time
    deadline = time.monotonic() + timeout
    try:
        pending = list(procs)
        while pending:
            for p in list(pending):
                rc = p.poll()
                if rc is None:
                    continue
                pending.remove(p)
                assert rc == 0, f"rank process exited with {rc}"
            assert time.monotonic() < deadline, "rank processes timed out"
            time.sleep(0.05)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
            p.wait()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [1, 2])
def test_exchange_matches_the_single_device_block(world, tmp_path, golden_dir):
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, str(HERE / "ep_worker.py"), str(r), str(world), str(port),
                               str(tmp_path / f"r{r}.npz")]) for r in range(world)]
    _wait_all(procs, 180)
    parts = [np.load(tmp_path / f"r{r}.npz") for r in range(world)]
    g = np.load(golden_dir / "moe.npz")
    assert np.array_equal(np.concatenate([p["ids"] for p in parts]), g["small_ids"])
    assert np.array_equal(np.concatenate([p["out"] for p in parts]), g["small_out"])
    if world > 1:
        assert all(int(p["sent"]) > 0 for p in parts)
