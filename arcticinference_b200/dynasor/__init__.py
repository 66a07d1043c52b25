"""Dynasor: early exit for reasoning models by probing how certain the model already is."""

from .certainty import (count_not_empty, equal_group, majority_voting, obtain_answer,  # noqa: F401
                        should_early_exit)
from .controller import DynasorController  # noqa: F401
from .math_equal import math_equal  # noqa: F401
