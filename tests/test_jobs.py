"""Fault-tolerant scheduling of the sharded pass: host-side only, failures made on the host
(a rank that stops between items), CPU processes over a TCPStore."""
import os
import sys
import time

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from voyager_compiler_b200.jobs import Manifest, WorkItem, checksum, run_items  # noqa: E402

ITEMS = [WorkItem(t, 0, 10 + t) for t in range(12)]


def _crc(item):
    return checksum(item.key.encode())


def _rank(rank, world, port, tmp, die_after, ret):
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=__import__("datetime").timedelta(seconds=60))
    done = []

    def work(item):
        if die_after is not None and rank == 1 and len(done) >= die_after:
            os._exit(17)                      # the rank vanishes holding a claimed item
        time.sleep(0.05)
        done.append(item.key)
        return _crc(item)

    man = Manifest(os.path.join(tmp, f"manifest_{rank}.json"))
    store.add("ready", 1)
    while store.add("ready", 0) < world:         # start together so that every rank gets items
        time.sleep(0.01)
    try:
        mine = run_items(store, rank, ITEMS, work, manifest=man, heartbeat_timeout=0.6, poll=0.05, give_up_after=30)
        ret[rank] = mine
        # keep the store's server alive until every survivor is through
        store.add("exited", 1)
        if rank == 0:
            t0 = time.time()
            while store.add("exited", 0) < world - (1 if die_after is not None else 0) and time.time() - t0 < 20:
                time.sleep(0.05)
    except Exception:  # noqa: BLE001
        import traceback
        ret[rank] = traceback.format_exc()


def _launch(tmp, die_after):
    world = 3
    port = 29800 + (os.getpid() % 150) + (0 if die_after is None else 1)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=_rank, args=(r, world, port, str(tmp), die_after, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(90)
            assert not p.is_alive()
        return dict(ret), [p.exitcode for p in procs]


def test_all_items_done_once_without_failures(tmp_path):
    ret, codes = _launch(tmp_path, None)
    assert codes == [0, 0, 0]
    keys = [k for r in ret.values() for k in r]
    assert sorted(keys) == sorted(i.key for i in ITEMS)


def test_items_of_a_vanished_rank_are_taken_over(tmp_path):
    ret, codes = _launch(tmp_path, 1)
    assert codes[1] == 17 and codes[0] == 0 and codes[2] == 0
    assert 1 not in ret
    keys = [k for r in (0, 2) for k in ret[r]]
    # the survivors finished everything the dead rank had not recorded
    man1 = Manifest(os.path.join(str(tmp_path), "manifest_1.json"))
    assert set(keys) | set(man1.done) == {i.key for i in ITEMS}


def test_manifest_resume_skips_finished_items(tmp_path):
    class Store(dict):
        def set(self, k, v): self[k] = v.encode() if isinstance(v, str) else v
        def get(self, k): return self[k]
        def check(self, ks): return all(k in self for k in ks)
        def add(self, k, n):
            self[k] = str((int(self[k]) if k in self else 0) + n).encode()
            return int(self[k])
        def compare_set(self, k, old, new):
            cur = self[k].decode() if k in self else ""
            if cur == old:
                self[k] = new.encode()
            return self[k]

    path = os.path.join(str(tmp_path), "m.json")
    calls = []
    man = Manifest(path)
    run_items(Store(), 0, ITEMS[:5], lambda it: calls.append(it.key) or _crc(it), manifest=man)
    assert len(calls) == 5 and len(Manifest(path).done) == 5
    calls.clear()
    man2 = Manifest(path)
    mine = run_items(Store(), 0, ITEMS, lambda it: calls.append(it.key) or _crc(it), manifest=man2)
    assert sorted(calls) == sorted(i.key for i in ITEMS[5:])      # only the unfinished ones ran
    assert len(Manifest(path).done) == len(ITEMS)
    assert Manifest(path).done[ITEMS[0].key]["crc"] == _crc(ITEMS[0])


def test_manifest_merges_the_other_ranks_files_on_resume(tmp_path):
    """One file per rank; a rerun sees what any rank finished, whichever rank gets the item this time."""
    p0, p1 = str(tmp_path / "manifest_0.json"), str(tmp_path / "manifest_1.json")
    m0, m1 = Manifest(p0), Manifest(p1)
    m0.record(ITEMS[0], 11, 0)
    m1.record(ITEMS[1], 22, 1)
    again = Manifest(p0, peers=str(tmp_path / "manifest_*.json"))
    assert again.finished(ITEMS[0]) and again.finished(ITEMS[1]) and not again.finished(ITEMS[2])
    assert again.done[ITEMS[1].key] == {"crc": 22, "rank": 1}
    again.record(ITEMS[2], 33, 0)                      # rewrites only its own file
    assert set(Manifest(p1).done) == {ITEMS[1].key}
    assert set(Manifest(p0).done) == {ITEMS[0].key, ITEMS[1].key, ITEMS[2].key}
    assert Manifest(p0, peers=[p1]).finished(ITEMS[1])


def test_waiting_rank_does_not_time_out_while_the_others_make_progress():
    """Phase 2: the pending set shrinking counts as progress even when this rank takes nothing."""
    class FakeStore:
        def __init__(self):
            self.d, self.t = {}, 0.0
        def set(self, k, v): self.d[k] = v.encode() if isinstance(v, str) else v
        def get(self, k): return self.d[k]
        def check(self, ks): return all(k in self.d for k in ks)
        def add(self, k, v):
            self.d[k] = str(int(self.d.get(k, b"0")) + v).encode()
            return int(self.d[k])
        def compare_set(self, k, old, new):
            cur = self.d.get(k, b"").decode()
            if cur == old:
                self.d[k] = new.encode()
            return self.d[k]

    store = FakeStore()
    items = ITEMS[:4]
    # another rank (7) has claimed everything and is alive; it finishes one item every 4 "seconds"
    store.add("next_item", len(items))
    for i in range(len(items)):
        store.set(f"claim/{i}", "7:0.0")
    finished = {"n": 0}

    def clock():
        store.t += 1.0
        store.set("hb/7", repr(store.t))
        if int(store.t) % 4 == 0 and finished["n"] < len(items):
            store.set(f"done/{finished['n']}", "7:1")
            finished["n"] += 1
        return store.t

    mine = run_items(store, 0, items, lambda it: 1, heartbeat_timeout=50.0, poll=0.0, give_up_after=6.0, clock=clock)
    assert mine == [] and finished["n"] == len(items)
