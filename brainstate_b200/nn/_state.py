"""Minimal state holders with the ``.value`` protocol the reference's layers use
(``brainstate._state.ParamState`` / ``FakeState``, ``brainstate/_state.py:1872,1897``).

Only what the event layers touch is provided: a ``value`` attribute that can be
read and assigned, and ``restore_value`` (used by the reference's JVP test,
``brainstate/nn/_event_fixedprob_test.py:106``).
"""
from __future__ import annotations


class State:
    __slots__ = ('_value',)

    def __init__(self, value):
        self._value = value

    @property
    def value(self):
        return self._value

    @value.setter
    def value(self, v):
        self._value = v

    def restore_value(self, v):
        self._value = v

    def __repr__(self):
        return f'{type(self).__name__}({self._value!r})'


class ParamState(State):
    """A trainable parameter."""
    __slots__ = ()


class FakeState(State):
    """A constant that looks like a state (zero-connection layers)."""
    __slots__ = ()
