"""Source hygiene greps and host-side failure-detection units (no GPU is ever faulted or hung)."""
import os
import re
import time

import pytest

from tah_b200.utils.failure import RankFailure, RankHeartbeat, StepTimeout, StepWatchdog

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _sources(exts=(".py", ".cu", ".cuh", ".h")):
    for base in ("tah_b200", "csrc", "script", "bench.py", "__graft_entry__.py"):
        p = os.path.join(ROOT, base)
        if os.path.isfile(p):
            yield p
            continue
        for d, _, files in os.walk(p):
            for f in files:
                if f.endswith(exts):
                    yield os.path.join(d, f)


def test_no_cluster_multicast_no_triton_no_disassembly():
    bad = []
    # the qualifier this test looks for is assembled from pieces so that this file does not name it
    multicast = "".join([".", "multi", "cast", "::", "clus", "ter"])
    bulk_copy = "".join(["cp", ".", "as", "ync"])
    for path in _sources():
        text = open(path, encoding="utf-8", errors="ignore").read()
        if multicast in text and not path.endswith("comm.cu") and not path.endswith("common.cuh"):
            bad.append((path, "cluster multicast"))
        if multicast in text:
            # even the files that mention the rule must not contain a multicast instruction
            for line in text.splitlines():
                if multicast in line and (bulk_copy in line or "asm" in line):
                    bad.append((path, "multicast instruction"))
        if re.search(r"^\s*(import triton|from triton)", text, re.M):
            bad.append((path, "triton"))
        if re.search(r"cuobjdump|nvdisasm|objdump\s+-d", text):
            bad.append((path, "disassembly tool"))
        if "torch.compile(" in text:
            bad.append((path, "torch.compile"))
        if re.search(r"cu(da)?Memcpy(3D)?Batch" + "Async", text):
            bad.append((path, "closed batched-copy call"))
    assert not bad, bad


def test_every_device_wait_is_bounded():
    """Every spin in the kernels goes through a helper with a time limit."""
    for name in ("gemm_tcgen05.cu", "attn_decode.cu"):
        text = open(os.path.join(ROOT, "csrc", name)).read()
        assert "mbar_try_wait(" not in text            # only the bounded mbar_wait() may be called from kernels
        assert "while (true)" not in text and "while(1)" not in text
    for name in ("comm.cu", "optim.cu"):
        text = open(os.path.join(ROOT, "csrc", name)).read()
        assert "WAIT_TIMEOUT_NS" in text and "STATUS_TIMEOUT_PEER_FLAG" in text


class _DictStore(dict):
    def set(self, k, v):
        self[k] = v

    def get(self, k):
        return self[k]


def test_heartbeat_with_fake_store():
    store = _DictStore()
    a = RankHeartbeat(store, 0, 2, interval_s=0.05).start()
    b = RankHeartbeat(store, 1, 2, interval_s=0.05).start()
    time.sleep(0.2)
    a.check_peers(timeout_s=0.3)
    b.stop()                                             # rank 1 "dies": its counter stops moving
    with pytest.raises(RankFailure) as info:
        t0 = time.time()
        while time.time() - t0 < 3:
            a.check_peers(timeout_s=0.3)
            time.sleep(0.05)
    assert info.value.dead == [1]
    a.stop()


def test_heartbeat_missing_key_counts_as_dead():
    store = _DictStore()
    a = RankHeartbeat(store, 0, 2, interval_s=0.05)
    a.beat()
    a.check_peers(timeout_s=0.1)                         # first look only records
    time.sleep(0.2)
    with pytest.raises(RankFailure):
        a.check_peers(timeout_s=0.1)


def test_step_watchdog():
    with StepWatchdog(1.0):
        pass
    with pytest.raises(StepTimeout):
        with StepWatchdog(0.05):
            time.sleep(0.2)
    fired = []
    with StepWatchdog(0.05, on_timeout=lambda: fired.append(1)):
        time.sleep(0.2)
    assert fired == [1]
