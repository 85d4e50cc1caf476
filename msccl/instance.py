"""Synthesis instance parameters (steps / rounds / chunks ...).

Parity: reference ``msccl/instance.py:6-39``.  ``str(instance)`` is part of
algorithm and file names, so its exact format is preserved.
"""
from dataclasses import dataclass, replace
from typing import Optional


@dataclass(frozen=True)
class Instance:
    steps: Optional[int]
    extra_rounds: int = 0
    chunks: int = 1
    pipeline: Optional[int] = None
    extra_memory: Optional[int] = None
    allow_exchange: bool = False

    def rounds(self) -> int:
        return self.steps + self.extra_rounds

    def set(self, **changes) -> 'Instance':
        """Copy with the given fields replaced; ``None`` values mean "keep"."""
        return replace(self, **{k: v for k, v in changes.items() if v is not None})

    def __str__(self) -> str:
        parts = [f'steps={self.steps}']
        if self.extra_rounds > 0:
            parts.append(f'rounds={self.rounds()}')
        if self.chunks > 1:
            parts.append(f'chunks={self.chunks}')
        if self.pipeline is not None:
            parts.append(f'pipeline={self.pipeline}')
        if self.extra_memory is not None:
            parts.append(f'extra_memory={self.extra_memory}')
        if self.allow_exchange:
            parts.append('allow_exchange')
        return ','.join(parts)
