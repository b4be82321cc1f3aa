"""``KernelManager`` (reference: ``src/mase_triton/manager.py:7-32``).

The reference toggles Triton's autotuner and reloads its kernel modules.  The CUDA kernels here are compiled
ahead of time, so most of them have nothing to tune at run time.  The one run-time choice is the CTA tile width
the weight of a tensor-core linear is packed for: with autotune enabled the layers time the candidate widths
on the GPU at their first call for an activation height and keep the fastest
(``mase_triton_b200.mxfp.gemm.choose_tile_rows``); disabled, the width with the least padded work is used.
"""

from __future__ import annotations

import logging

logger = logging.getLogger(__name__)


class KernelManager:
    _autotune_is_enabled = False
    _choices: dict = {}

    @classmethod
    def enable_autotune(cls) -> None:
        cls._autotune_is_enabled = True
        logger.info("Autotune enabled: tensor-core linears time their candidate tile widths at first use")

    @classmethod
    def disable_autotune(cls) -> None:
        cls._autotune_is_enabled = False
        logger.info("Autotune disabled")

    @classmethod
    def autotune_is_enabled(cls) -> bool:
        return cls._autotune_is_enabled

    @classmethod
    def record_choice(cls, what: tuple, choice, timings_ms: dict) -> None:
        """Called by the tuned paths: remembers what was chosen and the measured times it was chosen from."""
        cls._choices[what] = {"choice": choice, "ms": dict(timings_ms)}
        logger.info("autotune %s -> %s (%s)", what, choice, {k: round(v, 4) for k, v in timings_ms.items()})

    @classmethod
    def tuned_choices(cls) -> dict:
        """Every choice made so far: ``{(name, *problem): {"choice": ..., "ms": {candidate: time}}}``."""
        return dict(cls._choices)
