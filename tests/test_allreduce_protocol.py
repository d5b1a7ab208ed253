"""The synchronisation protocol of the one-shot peer-memory all-reduce, modelled on the host:
ranks are threads, regions and flags are shared arrays, every step of a rank is one statement
of the kernel (publish flag, wait for peers' flags with >=, read peers' slots, leave).  The model
checks the two claims the design rests on: with slots alternating between consecutive calls no
rank ever overwrites a slot a peer is still reading, and a peer that is one call ahead does not
stall or confuse a slow rank (flags are compared with >=, never ==)."""
import random
import threading
import time

import numpy as np
import pytest

from awq_b200 import tp


class Model:
    def __init__(self, world: int, width: int = 8):
        self.world = world
        self.flags = np.zeros((world, world), dtype=np.int64)        # flags[owner][writer]
        self.slots = np.zeros((world, 2, width), dtype=np.float64)   # slots[owner][slot]
        self.readers = np.zeros((world, 2), dtype=np.int64)          # peers reading slots[owner][slot]
        self.lock = threading.Lock()
        self.errors: list[str] = []

    def rank_main(self, rank: int, calls: int, rng: random.Random, results: list):
        for call in range(calls):
            epoch = call + 1
            slot = tp.slot_for_call(call)
            # the GEMM of this call writes the partial
            with self.lock:
                if self.readers[rank, slot] != 0:
                    self.errors.append(f"rank {rank} call {call}: slot {slot} overwritten while "
                                       f"{self.readers[rank, slot]} peer(s) read it")
                self.slots[rank, slot, :] = (rank + 1) * 1000 + call
            time.sleep(rng.random() * 0.002)
            # start barrier: publish, then wait for every peer with >=
            with self.lock:
                for peer in range(self.world):
                    if peer != rank:
                        self.flags[peer, rank] = epoch
            deadline = time.time() + 10
            while True:
                with self.lock:
                    ready = all(self.flags[rank, p] >= epoch for p in range(self.world) if p != rank)
                if ready:
                    break
                if time.time() > deadline:
                    self.errors.append(f"rank {rank} call {call}: wait ran out")
                    return
                time.sleep(0)
            # read every rank's slot, in rank order
            with self.lock:
                for p in range(self.world):
                    self.readers[p, slot] += 1
            time.sleep(rng.random() * 0.002)
            with self.lock:
                total = sum(self.slots[p, slot, 0] for p in range(self.world))
                for p in range(self.world):
                    self.readers[p, slot] -= 1
            results.append((rank, call, total))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_alternating_slots_are_never_overwritten_while_read(world):
    model = Model(world)
    calls = 40
    results: list = []
    threads = [threading.Thread(target=model.rank_main,
                                args=(r, calls, random.Random(r * 7 + world), results))
               for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert not model.errors, model.errors[:3]
    assert len(results) == world * calls
    for rank, call, total in results:
        assert total == sum((p + 1) * 1000 + call for p in range(world)), (rank, call, total)


def test_region_layout_and_slot_rule():
    off0, off1, size = tp.region_layout(16 * 8192 * 2)
    assert off0 == tp.FLAG_BYTES == 4096 and off0 % 16 == 0 and off1 % 16 == 0
    assert off1 - off0 >= 16 * 8192 * 2 and size - off1 >= 16 * 8192 * 2
    assert [tp.slot_for_call(i) for i in range(5)] == [0, 1, 0, 1, 0]
    # flags of 2 phases x 32 blocks x 8 ranks fit the flag area
    assert 2 * 32 * 8 * 4 <= tp.FLAG_BYTES
