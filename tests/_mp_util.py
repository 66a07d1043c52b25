"""Helpers for tests that run ranks as child processes."""

import os
import socket


def free_port():
    """A port for the ranks' rendezvous, taken from below the kernel's ephemeral range
    (32768 and up): a port handed out by bind(0) can be claimed as the local end of some
    other process's outgoing connection before rank 0 gets to listen on it."""
    import random
    rng = random.Random(os.getpid() * 7919 + int.from_bytes(os.urandom(4), "little"))
    for _ in range(200):
        p = rng.randrange(15000, 30000)
        s = socket.socket()
        try:
            s.bind(("127.0.0.1", p))
        except OSError:
            continue
        finally:
            s.close()
        return p
    raise RuntimeError("no free port found")


def result_or_child_failure(q, procs, timeout):
    """The first result a rank puts on ``q``; fails as soon as a rank has exited with an
    error instead of waiting out the whole timeout."""
    import queue as _queue
    import time
    deadline = time.time() + timeout
    while time.time() < deadline:
        try:
            return q.get(timeout=2)
        except _queue.Empty:
            bad = [(i, p.exitcode) for i, p in enumerate(procs) if p.exitcode not in (None, 0)]
            if bad:
                for p in procs:
                    if p.is_alive():
                        p.terminate()
                raise AssertionError("rank(s) exited with an error: %s" % bad)
    for p in procs:
        if p.is_alive():
            p.terminate()
    raise AssertionError("no result from the ranks within %d s" % timeout)
