"""Model of the two-slot flag protocol of the peer-memory collectives (parallel/symm.py,
ops/csrc/comm.cu) with one thread per rank: every use writes this rank's payload into slot
``use % 2``, raises this rank's flag word on every peer, waits until all of its own flag words
have reached ``use_count + 1`` and only then reads the peers' payloads. The claim under test is
the one the kernels rely on: with two alternating slots a payload is never overwritten before
every peer has read it, whatever the relative speed of the ranks."""
import random
import threading
import time


def _run(world: int, uses: int, seed: int):
    payload = [[None, None] for _ in range(world)]            # payload[rank][slot]
    flags = [[[0] * world for _ in range(2)] for _ in range(world)]   # flags[rank][slot][src]
    errors = []
    rng = random.Random(seed)
    delays = [[rng.random() * 2e-4 for _ in range(uses)] for _ in range(world)]

    def rank_main(r):
        use_count = [0, 0]
        for k in range(uses):
            s = k % 2
            time.sleep(delays[r][k])
            payload[r][s] = (r, k)                             # stage
            for peer in range(world):                          # signal every rank (release)
                flags[peer][s][r] += 1
            want = use_count[s] + 1
            t0 = time.time()
            while any(flags[r][s][src] < want for src in range(world)):   # bounded wait
                if time.time() - t0 > 10.0:
                    errors.append(f"rank {r} use {k}: wait ran out")
                    return
                time.sleep(0)
            time.sleep(delays[r][k] / 2)                       # a slow reader after the wait
            for peer in range(world):                          # consume
                got = payload[peer][s]
                if got != (peer, k):
                    errors.append(f"rank {r} use {k}: read {got} from rank {peer}")
            use_count[s] = want

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return errors


def test_two_slots_are_enough_for_any_interleaving():
    for world, seed in ((2, 0), (4, 1), (8, 2)):
        assert _run(world, 60, seed) == []


def test_one_slot_would_not_be(monkeypatch):
    """The same model with a single slot does lose payloads: the check has teeth."""
    world, uses = 2, 40
    payload = [None] * world
    flags = [[0] * world for _ in range(world)]
    bad = []

    def rank_main(r):
        for k in range(uses):
            if r == 1:
                time.sleep(2e-4)                               # rank 1 is always late
            payload[r] = (r, k)
            for peer in range(world):
                flags[peer][r] += 1
            while any(flags[r][src] < k + 1 for src in range(world)):
                time.sleep(0)
            if r == 1:
                time.sleep(2e-4)                               # ... also between wait and read
            for peer in range(world):
                if payload[peer] != (peer, k):
                    bad.append((r, k, payload[peer]))

    ts = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert bad, "a single slot is overwritten by the fast rank before the slow one has read it"
