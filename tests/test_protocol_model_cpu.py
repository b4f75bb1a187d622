"""CPU-thread model of the flag protocols the NVLink kernels use (no GPU): every "rank" is a thread, the
symmetric buffers are shared Python lists, peer stores / flag updates are ordinary writes under the GIL.

* exchange protocol of ``tp_topk_merge_kernel`` (``csrc/comm.cu``): deliver to every peer's slot ``[epoch
  parity][source]``, write the call's epoch into the peer's arrival word of this source, wait until all own
  words have reached the epoch, read.  (One counted word per rank is not enough: a fast peer's next call can
  complete the count while a slow peer's delivery is missing; an earlier form of the kernel had that race and
  this model showed it.)  The model checks that with two slots a reader never sees data of another call
  although peers run up to one call ahead, and that the wait is bounded: a rank that never delivers makes the others give up with a status
  instead of spinning forever.
* landing-flag protocol of the push all-gather (``shard_gather_push_kernel`` + the consumer's ``wait_peer_rows``):
  the consumer's target grows by the push grid size per use; a consumer never reads a buffer before all sources
  of THAT use have landed, and a producer never overwrites it before every consumer released the previous use.
"""
import random
import threading
import time


def _spin(cond, limit_s):
    t0 = time.monotonic()
    while not cond():
        if time.monotonic() - t0 > limit_s:
            return False
        time.sleep(0)
    return True


def _run_exchange(world, calls, absent=None, limit_s=5.0, seed=0):
    slots = [[[None] * world for _ in range(2)] for _ in range(world)]      # slots[rank][parity][source]
    arrive = [[0] * world for _ in range(world)]                           # arrive[rank][source] = epoch delivered
    status, bad = [0] * world, []

    def rank_main(r):
        rng = random.Random(seed * 100 + r)
        for ep in range(1, calls + 1):
            if absent == (r, ep):
                return                                                     # this rank leaves before call ep
            par = ep & 1
            for q in range(world):
                time.sleep(rng.random() * 1e-4)
                slots[q][par][r] = (ep, r)
                arrive[q][r] = ep                                          # release store, one word per source
            if not _spin(lambda: all(a >= ep for a in arrive[r]), limit_s):
                status[r] = 4                                              # STATUS_TIMEOUT_PEER_FLAG, then return
                return
            got = [slots[r][par][q] for q in range(world)]
            if got != [(ep, q) for q in range(world)]:
                bad.append((r, ep, got))
            time.sleep(rng.random() * 2e-4)                                # "merge" while peers may run ahead

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert not any(t.is_alive() for t in threads)
    return status, bad


def test_exchange_with_two_slots_never_mixes_calls():
    for world in (2, 4, 8):
        status, bad = _run_exchange(world, calls=40, seed=world)
        assert status == [0] * world and bad == []


def test_exchange_wait_is_bounded_when_a_rank_never_delivers():
    t0 = time.monotonic()
    status, bad = _run_exchange(4, calls=10, absent=(2, 6), limit_s=0.3)
    assert time.monotonic() - t0 < 10
    assert bad == []
    assert status[2] == 0 and all(status[r] == 4 for r in (0, 1, 3))      # the others report the timeout and return


def test_push_gather_flags_order_producers_and_consumers():
    world, grid, uses = 4, 3, 25
    buf = [[None] * world for _ in range(world)]                           # buf[rank][source]
    landed = [[0] * world for _ in range(world)]                           # landed[rank][source]: += 1 per CTA
    ready = [[0] * world for _ in range(world)]                            # ready[rank][source] = use released
    bad = []

    def rank_main(r):
        rng = random.Random(r)
        for use in range(1, uses + 1):
            # producer: "I am done reading the previous contents" to every peer, wait for theirs, then push
            for q in range(world):
                ready[q][r] = use
            assert _spin(lambda: all(ready[r][q] >= use for q in range(world)), 10.0)
            for cta in range(grid):
                time.sleep(rng.random() * 1e-4)
                for q in range(world):
                    buf[q][r] = use
                    landed[q][r] += 1
            # consumer: wait until every source's CTAs of THIS use have landed, then read
            assert _spin(lambda: all(landed[r][q] >= use * grid for q in range(world)), 10.0)
            got = list(buf[r])
            if any(g < use for g in got) or any(g > use for g in got):
                bad.append((r, use, got))
            time.sleep(rng.random() * 1e-4)

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert not any(t.is_alive() for t in threads) and bad == []
