"""Happens-before checker for the stream discipline of the executors.

Host and simulated-GPU streams append ``("record", stream, event)``,
``("wait", stream, event)`` and ``("sync", stream, -1)`` to ``stream.ORDER_LOG``
when logging is on.  ``check(log, accesses)`` verifies that every access to a
buffer on one stream is ordered after the last conflicting access on another
stream by a record -> wait chain (or a host sync), i.e. that the executor never
relies on timing.  Accesses are ``(position_in_log, stream_id, buffer_id,
is_write)``.  This is the host-side substitute for a device race detector."""
from __future__ import annotations

from .. import stream as _stream


class logging_streams(object):
    def __enter__(self):
        _stream.ORDER_LOG.clear()
        _stream.LOGGING[0] = True
        return _stream.ORDER_LOG

    def __exit__(self, *a):
        _stream.LOGGING[0] = False


def _clock_join(a, b):
    out = dict(a)
    for k, v in b.items():
        if out.get(k, -1) < v:
            out[k] = v
    return out


def check(log, accesses):
    """Returns a list of violations (empty = the schedule is race-free under the
    recorded dependencies).  Vector clocks per stream; events carry the clock of
    their recording stream."""
    clocks = {}                # stream -> {stream: counter}
    event_clock = {}
    acc_by_pos = {}
    for pos, s, buf, w in accesses:
        acc_by_pos.setdefault(pos, []).append((s, buf, w))
    last_write, last_reads, violations = {}, {}, []

    host = [{}]                # what the host has observed through stream syncs

    def tick(s):
        # anything submitted after a host sync is ordered after what that sync observed
        c = clocks[s] = _clock_join(clocks.get(s, {}), host[0])
        c[s] = c.get(s, 0) + 1
        return c

    def ordered(before_clock, s):
        cur = clocks.get(s, {})
        return all(cur.get(k, -1) >= v for k, v in before_clock.items())
    for pos, (kind, s, ev) in enumerate(log):
        # accesses listed at position `pos` happen just BEFORE log entry `pos`
        for (as_, buf, w) in acc_by_pos.get(pos, []):
            c = dict(tick(as_))
            lw = last_write.get(buf)
            if lw is not None and lw[0] != as_ and not ordered(lw[1], as_):
                violations.append(("unordered after write", buf, lw[0], as_, pos))
            if w:
                for rs, rc in last_reads.get(buf, []):
                    if rs != as_ and not ordered(rc, as_):
                        violations.append(("write unordered after read", buf, rs, as_, pos))
                last_write[buf] = (as_, c)
                last_reads[buf] = []
            else:
                last_reads.setdefault(buf, []).append((as_, c))
        if kind == "record":
            event_clock[ev] = dict(tick(s))
        elif kind == "wait":
            if ev in event_clock:
                clocks[s] = _clock_join(_clock_join(clocks.get(s, {}), host[0]), event_clock[ev])
        elif kind == "sync":
            host[0] = _clock_join(host[0], clocks.get(s, {}))
    return violations
