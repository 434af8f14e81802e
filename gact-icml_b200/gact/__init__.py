"""gact: activation-compressed training, B200-native.

Same Python surface as the GACT reference package (``gact/gact/__init__.py``): ``gact.config``,
``gact.set_optimization_level``, ``gact.set_adapt_interval``, ``gact.controller.Controller`` and
``gact.ops``.  All device work goes through ``libgact_b200.so`` (hand-written sm_100a kernels behind a C
ABI, bound with ctypes in ``gact._native``); there is no CPU fallback.
"""
from . import ops
from . import controller
from .conf import config, set_optimization_level, set_adapt_interval
from .controller import Controller

__all__ = ["ops", "controller", "config", "set_optimization_level", "set_adapt_interval", "Controller"]
