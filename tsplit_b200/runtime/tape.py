"""Record one step's native calls and replay them from C++ (``csrc/runtime/step_tape.cc``).

The executors drive the GPU through ``extern "C"`` entries only: kernels, event records, stream waits, copies
to and from pinned host memory.  Every such call passes through the library proxy
(``utils/launch_counter.CountingLib``), which hands it to the active :class:`Recorder`.  A planned step uses the
same addresses every time, so the recorded list IS the step; :class:`Tape` replays it with one foreign call, which
is what the reference's per-node Python loop (``python/athena/gpu_ops/executor.py:140-152``) becomes here.

Arguments that change from step to step are marked with :func:`dyn` at the call site; their values are supplied
at every replay.  A ``byref`` result (a count the entry computes on the host from the geometry) points into the
tape's own storage at replay.  A call with an argument that cannot be stored (a Python object, a ``POINTER``
instance) makes the recording invalid, and the executor stays on its Python loop.
"""
from __future__ import annotations

import ctypes
import struct
from ctypes import c_char_p, c_int, c_longlong, c_void_p

from .. import _base

ACTIVE = [None]

#: entries that are queries or graph control, never actions of a step
NOT_ACTIONS = {"tsb_graph_begin", "tsb_graph_end", "tsb_graph_launch", "tsb_graph_destroy", "tsb_mem_info",
               "tsb_scratch_bytes", "tsb_scratch_trim", "tsb_device_status", "tsb_comm_status"}

_INT32 = (ctypes.c_int, ctypes.c_short, ctypes.c_byte, ctypes.c_bool)
_UINT32 = (ctypes.c_uint, ctypes.c_ushort, ctypes.c_ubyte)
_INT64 = (ctypes.c_long, ctypes.c_longlong, ctypes.c_ulong, ctypes.c_ulonglong, ctypes.c_size_t, ctypes.c_ssize_t)


def available():
    lib = _base.runtime()
    lib.tsb_tape_available.restype = c_int
    return bool(lib.tsb_tape_available())


def dyn(key, value):
    """Mark ``value`` (a ctypes scalar about to be passed to an entry) as changing from step to step."""
    rec = ACTIVE[0]
    if rec is not None:
        rec._dyn_ids[id(value)] = key
        rec.keep.append(value)
    return value


def _encode(a):
    """(type code, 8-byte cell value, blob bytes or None) of one argument, or None if it cannot be stored."""
    if isinstance(a, c_void_p):
        return "p", int(a.value or 0), None
    if isinstance(a, _INT32):
        return "i", int(a.value) & 0xFFFFFFFF, None
    if isinstance(a, _UINT32):
        return "u", int(a.value) & 0xFFFFFFFF, None
    if isinstance(a, _INT64):
        return "q", int(a.value) & 0xFFFFFFFFFFFFFFFF, None
    if isinstance(a, ctypes.c_float):
        return "f", struct.unpack("<I", struct.pack("<f", a.value))[0], None
    if isinstance(a, ctypes.c_double):
        return "d", struct.unpack("<Q", struct.pack("<d", a.value))[0], None
    if a is None:
        return "p", 0, None
    if isinstance(a, bool):
        return "i", int(a), None
    if isinstance(a, int):
        if -2**31 <= a < 2**31:
            return "i", a & 0xFFFFFFFF, None          # what ctypes passes for a bare Python int
        return None
    if isinstance(a, (ctypes.Array, ctypes.Structure)):
        return "b", 0, bytes(a)
    if type(a).__name__ == "CArgObject" and isinstance(getattr(a, "_obj", None), ctypes._SimpleCData):
        # byref(result): the entry writes a host-computed value (a chunk count) there; at replay it writes the
        # same value into the tape's own copy
        return "b", 0, bytes(a._obj)
    return None


class Recorder(object):
    def __init__(self):
        self.fns, self.names, self.arg_begin = [], [], [0]
        self.types, self.values, self.dyn_slot = bytearray(), [], []
        self.blob = bytearray()
        self.dyn_keys = []              # slot -> key
        self.dyn_codes = []             # slot -> type code
        self._dyn_ids = {}
        self.keep = []                  # objects whose addresses the actions use (events, host buffers)
        self.kernels = 0
        self.invalid = None             # reason the recording cannot be replayed

    def record(self, name, cfunc, args, kernels):
        if name in NOT_ACTIONS or self.invalid is not None:
            return
        argtypes = getattr(cfunc, "argtypes", None)
        for i, a in enumerate(args):
            if argtypes and not isinstance(a, ctypes._SimpleCData) and not isinstance(a, (ctypes.Array, ctypes.Structure)) \
                    and a is not None and i < len(argtypes):
                try:
                    a = argtypes[i](a)
                except Exception:
                    pass
            enc = _encode(a)
            if enc is None:
                self.invalid = "%s: argument %d (%s) cannot be stored by value" % (name, i, type(a).__name__)
                return
            code, value, data = enc
            if data is not None:
                pad = (-len(self.blob)) % 16
                self.blob.extend(b"\0" * pad)
                value = len(self.blob)
                self.blob.extend(data)
            key = self._dyn_ids.get(id(args[i]))
            slot = -1
            if key is not None:
                if code == "b":
                    self.invalid = "%s: a by-pointer argument cannot change between steps" % name
                    return
                if key in self.dyn_keys:
                    slot = self.dyn_keys.index(key)
                else:
                    slot = len(self.dyn_keys)
                    self.dyn_keys.append(key)
                    self.dyn_codes.append(code)
            self.types.extend(code.encode())
            self.values.append(value)
            self.dyn_slot.append(slot)
        self.fns.append(ctypes.cast(cfunc, c_void_p).value)
        self.names.append(name)
        self.arg_begin.append(len(self.values))
        self.kernels += kernels

    def hold(self, obj):
        self.keep.append(obj)


class Tape(object):
    """A recorded step.  ``replay(values)`` runs it; ``values`` maps every dynamic key to a ctypes scalar."""

    def __init__(self, rec):
        assert rec.invalid is None, rec.invalid
        lib = _base.runtime()
        lib.tsb_tape_create.restype = c_void_p
        n = len(rec.fns)
        total = len(rec.values)
        self.names = list(rec.names)
        self.kernels = rec.kernels
        self.dyn_keys, self.dyn_codes = list(rec.dyn_keys), list(rec.dyn_codes)
        self.keep = rec.keep
        self.lib = lib
        self.handle = lib.tsb_tape_create(
            c_int(n), (c_void_p * max(n, 1))(*rec.fns), (c_int * (n + 1))(*rec.arg_begin),
            c_char_p(bytes(rec.types)), (ctypes.c_uint64 * max(total, 1))(*rec.values),
            (c_int * max(total, 1))(*rec.dyn_slot), c_int(len(rec.dyn_keys)),
            (ctypes.c_ubyte * max(len(rec.blob), 1)).from_buffer_copy(bytes(rec.blob) or b"\0"),
            c_longlong(len(rec.blob)))
        if not self.handle:
            raise RuntimeError("the native step tape could not be built (libffi missing or an unsupported argument)")
        self.last_host_ns = 0

    def __len__(self):
        return len(self.names)

    def replay(self, values=None, first=0, last=None):
        """Run actions [first, last).  Returns None, or raises ``TapeError`` carrying the failing entry's name and status."""
        values = values or {}
        cells = []
        for key, code in zip(self.dyn_keys, self.dyn_codes):
            enc = _encode(values[key])
            assert enc is not None and enc[0] == code, "dynamic argument %r changed type" % (key,)
            cells.append(enc[1])
        failed, ns = c_int(-1), c_longlong(0)
        rc = self.lib.tsb_tape_replay(c_void_p(self.handle), c_int(first), c_int(len(self.names) if last is None else last),
                                      (ctypes.c_uint64 * max(len(cells), 1))(*cells), c_int(len(cells)),
                                      ctypes.byref(failed), ctypes.byref(ns))
        self.last_host_ns = ns.value
        if rc:
            name = self.names[failed.value] if 0 <= failed.value < len(self.names) else "?"
            raise TapeError(name, rc, failed.value)

    def __del__(self):
        try:
            if self.handle:
                self.lib.tsb_tape_destroy(c_void_p(self.handle))
                self.handle = None
        except Exception:
            pass


class TapeError(RuntimeError):
    def __init__(self, name, status, index):
        RuntimeError.__init__(self, "%s (action %d of the recorded step) failed: %s" % (
            name, index, _base.error_string(status)))
        self.entry, self.status, self.index = name, status, index


class recording(object):
    """``with recording() as rec:`` every proxied native call made inside is appended to ``rec``."""

    def __enter__(self):
        assert ACTIVE[0] is None, "a step is already being recorded"
        self.rec = ACTIVE[0] = Recorder()
        return self.rec

    def __exit__(self, *a):
        ACTIVE[0] = None
