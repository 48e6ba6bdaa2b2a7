"""Parameter checkpointing in the reference's on-disk format.

``Saver(file).append(key, value); .save()`` writes ONE pickled ``dict``;
``Loader(file).load(key)`` reads it back (``python/athena/model.py:6-48``).
Files written by the Python-2 reference (pickle protocol 0/2) load here through
``encoding='latin1'``.  Optional extra keys (``__optimizer__/<var>/<slot>``,
``__step__``) carry optimizer state; loaders that do not know them ignore them.
"""
from __future__ import annotations

import pickle

import numpy as np

from . import ndarray


class Saver(object):
    def __init__(self, file_path, protocol=2):
        self.file_path = file_path
        self.protocol = protocol
        self.params = {}

    def append(self, key, value):
        if isinstance(value, ndarray.NDArray):
            value = value.asnumpy()
        self.params[key] = np.asarray(value) if not np.isscalar(value) else value

    def append_variables(self, nodes):
        """Convenience: one entry per variable node, keyed by its name."""
        for n in nodes:
            self.append(n.name, n.tensor_value)

    def append_optimizer(self, optimizer):
        for k, v in optimizer.state_dict().items():
            self.params[k] = v

    def save(self):
        with open(self.file_path, "wb") as f:
            pickle.dump(self.params, f, protocol=self.protocol)


class Loader(object):
    def __init__(self, file_path):
        self.file_path = file_path
        with open(file_path, "rb") as f:
            try:
                self.params = pickle.load(f)
            except UnicodeDecodeError:
                f.seek(0)
                self.params = pickle.load(f, encoding="latin1")

    def load(self, key):
        return self.params[key]

    def keys(self):
        return list(self.params.keys())

    def restore_variables(self, nodes, ctx=None):
        for n in nodes:
            v = np.asarray(self.params[n.name], dtype=np.float32)
            if isinstance(n.tensor_value, ndarray.NDArray):
                n.tensor_value._sync_copyfrom(v)
            else:
                n.tensor_value = v if ctx is None else ndarray.array(v, ctx, use_pool=False)

    def restore_optimizer(self, optimizer):
        optimizer.load_state_dict(self.params)
