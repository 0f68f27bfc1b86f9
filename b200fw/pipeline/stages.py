"""Layer-to-stage assignment (remainder layers go to the first stages) and the per-rank stage view
(src/distributed/pipeline_parallel.py:23-150)."""
from __future__ import annotations

from typing import List, Optional, Tuple

from ..dist.context import ParallelContext


def split_layers_to_stages(num_layers: int, pp_size: int) -> List[Tuple[int, int]]:
    """``[start, end)`` per stage; the ``num_layers % pp_size`` extra layers go to the first stages.  With fewer
    layers than stages the last stages are empty (``(n, n)``), as in the reference; the engine refuses such a
    layout when it builds the model."""
    assert pp_size >= 1 and num_layers >= 0
    base, extra = divmod(num_layers, pp_size)
    out, start = [], 0
    for s in range(pp_size):
        n = base + (1 if s < extra else 0)
        out.append((start, start + n))
        start += n
    return out


class PipelineParallelContext:
    def __init__(self, *args, num_layers: Optional[int] = None, ctx: Optional[ParallelContext] = None,
                 pp_size: Optional[int] = None, pp_rank: Optional[int] = None,
                 parallel_context: Optional[ParallelContext] = None):
        """``PipelineParallelContext(num_layers, ctx)`` or, in the reference's order,
        ``PipelineParallelContext(parallel_context, num_layers)``; ``pp_size`` / ``pp_rank`` override the context's
        (or stand in for it when there is none)."""
        for a in args:
            if isinstance(a, ParallelContext):
                ctx = a
            elif isinstance(a, int) and num_layers is None:
                num_layers = a
            elif isinstance(a, int) and pp_size is None:
                pp_size = a
            elif isinstance(a, int):
                pp_rank = a
        ctx = ctx if ctx is not None else parallel_context
        assert isinstance(num_layers, int), "PipelineParallelContext needs num_layers"
        self.ctx = ctx
        self.pp_size = pp_size if pp_size is not None else (ctx.pp_size if ctx else 1)
        self.pp_rank = pp_rank if pp_rank is not None else (ctx.pp_rank if ctx else 0)
        self.stages = split_layers_to_stages(num_layers, self.pp_size)
        self.layer_start, self.layer_end = self.stages[self.pp_rank]

    @property
    def num_local_layers(self) -> int:
        return self.layer_end - self.layer_start

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    @property
    def prev_rank(self) -> Optional[int]:
        return None if self.ctx is None else self.ctx.pp_prev_rank

    @property
    def next_rank(self) -> Optional[int]:
        return None if self.ctx is None else self.ctx.pp_next_rank

    @property
    def group(self):
        return None if self.ctx is None else self.ctx.pp_group

    def local_to_global(self, i: int) -> int:
        return self.layer_start + i

    # ---- the reference's property names (src/distributed/pipeline_parallel.py:96-143) -------------------------
    @property
    def pp_group(self):
        return self.group

    @property
    def stage_layer_range(self) -> Tuple[int, int]:
        """Layers ``[start, end)`` of this stage."""
        return self.layer_start, self.layer_end

    @property
    def num_layers_this_stage(self) -> int:
        return self.num_local_layers
