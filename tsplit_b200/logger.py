"""Process-wide logger writing to ``<name>.log`` and to the console
(reference: ``python/athena/logger.py:3-26``)."""
from __future__ import annotations

import logging

_instances = {}


class Logger(object):
    def __new__(cls, name="tsplit_b200", level=logging.INFO, to_file=True):
        if name in _instances:
            return _instances[name]
        self = object.__new__(cls)
        self.logger = logging.getLogger(name)
        self.logger.setLevel(level)
        fmt = logging.Formatter("%(asctime)s %(levelname)s %(message)s")
        if not self.logger.handlers:
            if to_file:
                fh = logging.FileHandler(name + ".log")
                fh.setFormatter(fmt)
                self.logger.addHandler(fh)
            sh = logging.StreamHandler()
            sh.setFormatter(fmt)
            self.logger.addHandler(sh)
        _instances[name] = self
        return self

    def info(self, *a):
        self.logger.info(*a)

    def debug(self, *a):
        self.logger.debug(*a)

    def warning(self, *a):
        self.logger.warning(*a)

    def error(self, *a):
        self.logger.error(*a)
