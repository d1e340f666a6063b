"""Event-connection layers (the part of ``brainstate.nn`` this package covers:
``brainstate/nn/__init__.py:54-59``)."""
from ._event_fixedprob import (FixedNumConn, EventFixedNumConn, EventFixedProb,
                               init_indices_without_replace, fixed_num_indices)
from ._event_linear import EventLinear
from ._delay import Delay, SpikeDelay, StateWithDelay
from ._state import ParamState, FakeState, State
from ._module import Module

__all__ = ['FixedNumConn', 'EventFixedNumConn', 'EventFixedProb', 'EventLinear', 'Delay', 'SpikeDelay', 'StateWithDelay',
           'init_indices_without_replace', 'fixed_num_indices', 'ParamState', 'FakeState', 'State', 'Module']
