"""Privacy accounting: process algebra, budgets, calibration, and the native PLD engine (torch-free)."""
from . import amplification, budgets, calibration, codec, core, discretization  # noqa: F401
from .accountant import Accountant  # noqa: F401
from .budgets import (advantage_budget, beta_budget, delta_budget, epsilon_budget, register_budget_serializer,  # noqa: F401
                      risk_budget)
from .calibration import CalibrateResult, calibrate  # noqa: F401
from .core import (CachedProcess, Composed, DpHorizonProcess, DpProcess, EpsDelta, Identity, NonPrivate, Repeated,  # noqa: F401
                   cached, compose, eps_delta, identity, nonprivate, repeat)
from .discretization import get_discretization, set_discretization  # noqa: F401

composition = core
mechanisms = core
