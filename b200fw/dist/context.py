"""3-D (dp x pp x tp) process-group layout.

Rank layout (the same as the reference, src/distributed/parallel_context.py:79):
``global_rank = dp_rank * (pp * tp) + pp_rank * tp + tp_rank``; TP groups are contiguous runs of
``tp`` ranks, PP groups stride by ``tp``, DP groups stride by ``pp * tp``
(src/distributed/parallel_context.py:137-172).  One process drives one GPU; NCCL is the backend on
GPUs, gloo on CPUs.  With world size 1 every group is ``None`` and all collectives are no-ops.
"""
from __future__ import annotations

import datetime
import os
from typing import List, Optional

import torch
import torch.distributed as dist


class ParallelContext:
    _instance: Optional["ParallelContext"] = None

    def __init__(self, tp_size=1, dp_size=1, pp_size=1, rank=0, world_size=1, local_rank=0,
                 backend="gloo", tp_group=None, dp_group=None, pp_group=None):
        """Plain construction describes one rank's coordinates; ``init_distributed`` / ``init_single_process``
        create the process groups.  Ready-made groups may be handed in (the reference's constructor takes
        ``tp_size, tp_group, dp_size, dp_group, pp_size, pp_group``: src/distributed/parallel_context.py:38-66)."""
        self.tp_size, self.dp_size, self.pp_size = tp_size, dp_size, pp_size
        self.global_rank, self.world_size, self.local_rank = rank, world_size, local_rank
        self.backend = backend
        self.tp_rank = rank % tp_size
        self.pp_rank = (rank // tp_size) % pp_size
        self.dp_rank = rank // (tp_size * pp_size)
        self.tp_group, self.pp_group, self.dp_group = tp_group, pp_group, dp_group
        self.pp_fwd_group = self.pp_bwd_group = None      # per-direction pipeline communicators (init_distributed)
        self.tp_ranks: List[int] = [rank]
        self.pp_ranks: List[int] = [rank]
        self.dp_ranks: List[int] = [rank]
        self.owns_process_group = False

    # ---- layout arithmetic (pure; also used by tests without any process group) --------------
    @staticmethod
    def coords(rank: int, tp: int, pp: int):
        return rank // (tp * pp), (rank // tp) % pp, rank % tp  # dp, pp, tp

    @staticmethod
    def group_table(world: int, tp: int, dp: int, pp: int):
        """All TP / PP / DP rank lists of a world, in creation order."""
        assert tp * dp * pp == world, f"tp*dp*pp={tp*dp*pp} != world_size={world}"
        tp_groups = [list(range(s, s + tp)) for s in range(0, world, tp)]
        pp_groups = [[d * pp * tp + p * tp + t for p in range(pp)] for d in range(dp) for t in range(tp)]
        dp_groups = [[d * pp * tp + p * tp + t for d in range(dp)] for p in range(pp) for t in range(tp)]
        return tp_groups, pp_groups, dp_groups

    # ---- construction --------------------------------------------------------------------------
    @classmethod
    def init_distributed(cls, tp_size=1, dp_size=1, pp_size=1, backend: Optional[str] = None,
                         timeout_s: float = 1800.0, init_single_process: bool = False) -> "ParallelContext":
        """Reads RANK / WORLD_SIZE / LOCAL_RANK, creates the process group if none exists and the tp / pp / dp
        sub-groups.  ``init_single_process=True`` (the reference's flag, src/distributed/parallel_context.py:94-130)
        returns the one-rank context when the job has a single process."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if init_single_process and world == 1 and tp_size * dp_size * pp_size == 1:
            return cls.init_single_process()
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if tp_size * dp_size * pp_size != world:
            raise ValueError(f"tp({tp_size})*dp({dp_size})*pp({pp_size}) != WORLD_SIZE({world})")
        if torch.cuda.is_available() and backend == "nccl":
            torch.cuda.set_device(local_rank % torch.cuda.device_count())
        ctx = cls(tp_size, dp_size, pp_size, rank, world, local_rank, backend)
        if world > 1:
            if not dist.is_initialized():
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", "29500")
                kwargs = {}
                if backend == "nccl":
                    kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
                dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                        timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
                ctx.owns_process_group = True
            tp_groups, pp_groups, dp_groups = cls.group_table(world, tp_size, dp_size, pp_size)
            # every rank must create every group, in the same order
            for ranks in tp_groups:
                g = dist.new_group(ranks) if tp_size > 1 else None
                if rank in ranks:
                    ctx.tp_group, ctx.tp_ranks = g, ranks
            for ranks in pp_groups:
                g = dist.new_group(ranks) if pp_size > 1 else None
                # one more communicator per direction of the pipeline (activations downstream, gradients upstream):
                # the two flows then never queue behind each other and each can be posted ahead of its use
                gf = dist.new_group(ranks) if pp_size > 1 else None
                gb = dist.new_group(ranks) if pp_size > 1 else None
                if rank in ranks:
                    ctx.pp_group, ctx.pp_ranks = g, ranks
                    ctx.pp_fwd_group, ctx.pp_bwd_group = gf, gb
            for ranks in dp_groups:
                g = dist.new_group(ranks) if dp_size > 1 else None
                if rank in ranks:
                    ctx.dp_group, ctx.dp_ranks = g, ranks
        cls._instance = ctx
        return ctx

    @classmethod
    def init_single_process(cls) -> "ParallelContext":
        ctx = cls(1, 1, 1, 0, 1, 0, "none")
        cls._instance = ctx
        return ctx

    @classmethod
    def get_instance(cls) -> "ParallelContext":
        if cls._instance is None:
            cls._instance = cls.init_single_process()
        return cls._instance

    @classmethod
    def reset(cls):
        cls._instance = None

    # ---- the reference's property names (src/distributed/parallel_context.py:239-286) -----------------------
    @property
    def rank(self) -> int:
        return self.global_rank

    @property
    def prev_rank(self) -> Optional[int]:
        """Global rank of the previous pipeline stage (``rank - tp_size``); ``None`` on the first stage."""
        return self.pp_prev_rank

    @property
    def next_rank(self) -> Optional[int]:
        return self.pp_next_rank

    def on_destroy(self, fn):
        """Run ``fn()`` before the process groups are torn down (``destroy``).  CUDA graphs that captured
        collectives must be released first: a communicator waits for every graph that references it."""
        self.__dict__.setdefault("_destroy_callbacks", []).append(fn)

    def destroy(self):
        for fn in reversed(self.__dict__.pop("_destroy_callbacks", [])):
            try:
                fn()
            except Exception:  # noqa: BLE001 - teardown goes on
                pass
        if self.owns_process_group and dist.is_initialized():
            dist.destroy_process_group()
        ParallelContext._instance = None

    # ---- properties ----------------------------------------------------------------------------
    @property
    def device(self) -> torch.device:
        if torch.cuda.is_available() and self.backend in ("nccl", "none"):
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    @property
    def is_first_pp_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_pp_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    @property
    def pp_prev_rank(self) -> Optional[int]:
        return None if self.is_first_pp_stage else self.global_rank - self.tp_size

    @property
    def pp_next_rank(self) -> Optional[int]:
        return None if self.is_last_pp_stage else self.global_rank + self.tp_size

    @property
    def is_main(self) -> bool:
        return self.global_rank == 0

    def barrier(self):
        if self.world_size > 1 and dist.is_initialized():
            dist.barrier()

    def __repr__(self):
        return (f"ParallelContext(rank={self.global_rank}/{self.world_size}, tp={self.tp_rank}/{self.tp_size}, "
                f"pp={self.pp_rank}/{self.pp_size}, dp={self.dp_rank}/{self.dp_size}, backend={self.backend})")
