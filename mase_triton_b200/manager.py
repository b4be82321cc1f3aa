"""``KernelManager`` kept for API compatibility (reference: ``src/mase_triton/manager.py:7-32``).

The reference toggles Triton's autotuner and reloads its kernel modules.  The CUDA
kernels here are compiled ahead of time with fixed launch shapes, so there is nothing
to tune at run time: the switch only records the flag.
"""

from __future__ import annotations

import logging

logger = logging.getLogger(__name__)


class KernelManager:
    _autotune_is_enabled = False

    @classmethod
    def enable_autotune(cls) -> None:
        cls._autotune_is_enabled = True
        logger.info("Autotune enabled (no effect: kernels are precompiled)")

    @classmethod
    def disable_autotune(cls) -> None:
        cls._autotune_is_enabled = False
        logger.info("Autotune disabled")

    @classmethod
    def autotune_is_enabled(cls) -> bool:
        return cls._autotune_is_enabled
