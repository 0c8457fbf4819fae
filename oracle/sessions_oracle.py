"""CPU restatement of the callers that drive the cache — TEST INFRASTRUCTURE ONLY.

Pure Python (small cases) over the C oracle's sequences.  Restates
combs-runtime/src/engine.rs: ``common_prefix`` :386-388 (pinned by the reference's own cases,
:1786-1794), ``SessionSet`` :266-314, the longest-common-prefix reuse :1257-1287, the
speculative acceptance and rollback :1476-1493, and the session snapshot :1541-1568.
One difference that the product shares: sessions are sequences of one arena instead of caches
with private arenas, so a dropped session's pages return to the common free-list.
"""
from __future__ import annotations

MAX_SESSIONS = 4  # engine.rs:243


def common_prefix(a, b) -> int:  # engine.rs:386-388
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


class OracleSessionSet:
    def __init__(self, arena, max_sessions: int = MAX_SESSIONS):
        self.arena, self.max_sessions = arena, max_sessions
        self.map: dict[str, dict] = {}
        self.tick = 0
        self.evictions = 0

    def acquire(self, key, prompt, reuse=True):  # engine.rs:1257-1287
        assert len(prompt) >= 1
        key = key or ""
        if reuse and key in self.map:
            s = self.map.pop(key)                                   # sessions.take
            shared = min(common_prefix(s["history"], prompt), len(prompt) - 1)
            if shared > 0:
                need = len(s["history"]) - shared
                popped = s["seq"].popn(need)
                if popped == need:
                    return s["seq"], shared
            s["seq"].close()
        return self.arena.new_seq(), 0

    def release(self, key, seq, history, reuse=True):  # engine.rs:1541-1568, put :296-313
        key = key or ""
        if not reuse:
            seq.close()
            return
        assert seq.seq_len() == len(history)
        old = self.map.pop(key, None)
        if old is not None and old["seq"] is not seq:
            old["seq"].close()
        self.tick += 1
        self.map[key] = {"history": list(history), "seq": seq, "last_used": self.tick}
        if len(self.map) > self.max_sessions:
            oldest = min(self.map, key=lambda k: self.map[k]["last_used"])
            self.map.pop(oldest)["seq"].close()
            self.evictions += 1

    def clear_all(self) -> int:  # engine.rs:287-291
        n = len(self.map)
        for k in sorted(self.map, key=lambda x: x.encode()):  # the reference's HashMap order is unspecified: by key here
            self.map[k]["seq"].close()
        self.map.clear()
        return n


def spec_verify_rollback(seq, draft, argmax):  # engine.rs:1476-1493
    k = len(draft)
    accepted = 0
    while accepted < k and argmax[accepted] == draft[accepted]:
        accepted += 1
    correction = argmax[min(accepted, k)]
    unwanted = k - accepted
    if unwanted > 0:
        popped = seq.popn(unwanted)
        if popped != unwanted:
            raise RuntimeError(f"speculative rollback popped {popped} of {unwanted} rows")
    return accepted, correction
