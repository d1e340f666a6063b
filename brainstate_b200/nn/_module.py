"""The sliver of ``brainstate.nn.Module`` the event layers rely on
(``brainstate/nn/_module.py:83-260``): a name, ``in_size``/``out_size`` normalised
to tuples, and ``__call__`` forwarding to ``update``."""
from __future__ import annotations

from typing import Optional, Sequence, Union

Size = Union[int, Sequence[int]]


def _as_size(v) -> tuple:
    if isinstance(v, (int,)):
        return (int(v),)
    return tuple(int(s) for s in v)


class Module:
    def __init__(self, name: Optional[str] = None):
        self.name = name
        self._in_size = None
        self._out_size = None

    @property
    def in_size(self):
        return self._in_size

    @in_size.setter
    def in_size(self, v):
        self._in_size = _as_size(v)

    @property
    def out_size(self):
        return self._out_size

    @out_size.setter
    def out_size(self, v):
        self._out_size = _as_size(v)

    def update(self, *args, **kwargs):
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.update(*args, **kwargs)
