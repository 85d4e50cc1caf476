"""msccl: programmable collectives for B200 - MSCCLang DSL and compiler, SMT synthesizer, plan
registry, CLI, and a native sm_100a executor (``msccl.runtime``) for MSCCL-IR XML.

Top-level names match the reference package (``msccl/__init__.py:4-6``).
"""
from msccl.autosynth import Collective, init, ndv2_perm, print_plans, tabulate_plans  # noqa: F401

__version__ = '3.0.0'
