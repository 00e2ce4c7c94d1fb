"""Fault-tolerant, resumable scheduling of the sharded whole-model quantization pass.

The data path needs no collective (every tensor, row and block is independent), so the only shared
state is *which work items are finished*.  That state lives in a key-value store
(``torch.distributed.TCPStore`` or any object with ``set/get/add/compare_set/check``) and in a
manifest file:

* work items are claimed dynamically (``store.add`` on a counter), which also balances load;
* every rank publishes a heartbeat between items; an item whose claimant stopped beating and that
  has no ``done`` record is re-claimed by a survivor with ``compare_set``, so a rank that raises,
  exits or never joins only costs the items it held;
* finished items are recorded in a JSON manifest with a checksum; a rerun skips them.

Failures are detected on the host, between kernel launches; nothing here waits on a GPU.
"""
from __future__ import annotations

import json
import os
import time
import zlib
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

__all__ = ["WorkItem", "Manifest", "run_items", "checksum"]


@dataclass(frozen=True)
class WorkItem:
    """Rows ``[row_begin, row_end)`` of tensor ``tensor``."""
    tensor: int
    row_begin: int
    row_end: int

    @property
    def key(self) -> str:
        return f"{self.tensor}:{self.row_begin}:{self.row_end}"


def checksum(*buffers: bytes) -> int:
    """CRC-32 over the concatenation of the given byte strings."""
    c = 0
    for b in buffers:
        c = zlib.crc32(b, c)
    return c & 0xFFFFFFFF


class Manifest:
    """``{item key: {"crc": int, "rank": int}}`` persisted as JSON with atomic replace.

    ``path`` is this rank's own file (one writer per file: a rewrite never loses another rank's records).
    ``peers`` are the other ranks' files, or a glob pattern that matches them; their records are merged in when
    the manifest is opened, so that a rerun skips what ANY rank finished, however the items were dealt the
    first time."""

    def __init__(self, path: Optional[str], peers: Optional[object] = None):
        self.path = path
        self.done: Dict[str, dict] = {}
        paths = [path] if path else []
        if isinstance(peers, str):
            import glob
            paths += sorted(glob.glob(peers))
        elif peers:
            paths += list(peers)
        for p in paths:
            if p and os.path.exists(p):
                try:
                    with open(p) as f:
                        self.done.update(json.load(f).get("done", {}))
                except (OSError, ValueError):
                    continue                     # a peer's file that is being replaced right now: its records come next time

    def record(self, item: WorkItem, crc: int, rank: int) -> None:
        self.done[item.key] = {"crc": int(crc), "rank": int(rank)}
        self.flush()

    def flush(self) -> None:
        if not self.path:
            return
        tmp = f"{self.path}.tmp.{os.getpid()}"
        with open(tmp, "w") as f:
            json.dump({"done": self.done}, f)
        os.replace(tmp, self.path)

    def finished(self, item: WorkItem) -> bool:
        return item.key in self.done


def _get(store, key: str) -> Optional[bytes]:
    return store.get(key) if store.check([key]) else None


def run_items(store, rank: int, items: Sequence[WorkItem], work: Callable[[WorkItem], int], *,
              manifest: Optional[Manifest] = None, heartbeat_timeout: float = 5.0, poll: float = 0.05,
              give_up_after: float = 600.0, clock: Callable[[], float] = time.time) -> List[str]:
    """Process ``items`` cooperatively with the other ranks sharing ``store``.

    ``work(item)`` does the quantization of one item (launch, synchronise, write the outputs) and
    returns a checksum.  Returns the keys this rank completed.  Every rank returns once all items
    are done, or raises ``TimeoutError`` after ``give_up_after`` seconds without progress."""
    mine: List[str] = []
    n = len(items)

    def beat():
        store.set(f"hb/{rank}", repr(clock()))

    def is_done(i: int) -> bool:
        return store.check([f"done/{i}"])

    def finish(i: int, crc: int):
        store.set(f"done/{i}", f"{rank}:{crc}")
        if manifest is not None:
            manifest.record(items[i], crc, rank)
        mine.append(items[i].key)

    def claimant_alive(claim: bytes) -> bool:
        r = claim.decode().split(":")[0]
        hb = _get(store, f"hb/{r}")
        return hb is not None and clock() - float(hb.decode()) <= heartbeat_timeout

    def run(i: int):
        beat()
        if manifest is not None and manifest.finished(items[i]):
            store.set(f"done/{i}", f"{rank}:{manifest.done[items[i].key]['crc']}")
            return
        finish(i, work(items[i]))
        beat()

    beat()
    # phase 1: dynamic claiming
    while True:
        i = store.add("next_item", 1) - 1
        if i >= n:
            break
        store.set(f"claim/{i}", f"{rank}:{clock()!r}")
        run(i)
    # phase 2: wait for stragglers, take over items whose claimant stopped beating
    last_progress = phase2_start = clock()
    n_pending = n + 1
    while True:
        beat()
        pending = [i for i in range(n) if not is_done(i)]
        if not pending:
            return mine
        if len(pending) < n_pending:             # the peers are getting on: slow is not stuck
            n_pending = len(pending)
            last_progress = clock()
        took = False
        for i in pending:
            claim = _get(store, f"claim/{i}")
            if claim is not None and claimant_alive(claim):
                continue
            if claim is None and clock() - phase2_start <= heartbeat_timeout:
                continue        # its owner may be between drawing the index and publishing the claim
            new = f"{rank}:{clock()!r}"
            old = claim.decode() if claim is not None else ""
            got = store.compare_set(f"claim/{i}", old, new)
            if got.decode() == new and not is_done(i):
                run(i)
                took = True
        if took:
            last_progress = clock()
        elif clock() - last_progress > give_up_after:
            raise TimeoutError(f"rank {rank}: items {pending} made no progress for {give_up_after} s")
        else:
            time.sleep(poll)
