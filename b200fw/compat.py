"""Import aliases for code written against the reference's package layout.

The reference is imported as ``src.<area>.<module>`` (``from src.engines.train_engine import TrainEngine``,
``from src.transfer.swift_sync import DoubleBufferedLoRA``: src/__init__.py and the sub-packages' ``__init__``
files).  This framework's modules are organised differently (``b200fw.train.engine``, ``b200fw.sync``, ...) but keep
the reference's class, function and field names, so an alias per module is enough to run such code unchanged::

    import b200fw.compat
    b200fw.compat.install()          # once, before the first ``import src...``
    from src.engines.train_engine import TrainEngine, TrainConfig

``install()`` registers a finder for the ``src`` name space; every ``src.X`` module is created on first import as a
view over the one or several ``b200fw`` modules listed in :data:`ALIASES` (their public names, earlier entries win).
Nothing of the reference is imported or needed.  If a real ``src`` package is already importable, ``install()`` leaves
it alone unless ``force=True``.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys
import types
from typing import Dict, List, Tuple

def kwarg_aliases(**aliases: str):
    """Decorator: ``@kwarg_aliases(state_dict="state")`` lets a function whose parameter is ``state`` also be called
    with the reference's keyword ``state_dict=``.  Giving both spellings of one parameter is an error."""
    import functools

    def wrap(fn):
        @functools.wraps(fn)
        def inner(*args, **kwargs):
            for theirs, ours in aliases.items():
                if theirs in kwargs:
                    if ours in kwargs:
                        raise TypeError(f"{fn.__name__}() got both {theirs!r} and {ours!r}")
                    kwargs[ours] = kwargs.pop(theirs)
            return fn(*args, **kwargs)
        return inner
    return wrap


# reference module -> modules of this package that provide its names
ALIASES: Dict[str, Tuple[str, ...]] = {
    "src.distributed.parallel_context": ("b200fw.dist.context",),
    "src.distributed.comm": ("b200fw.dist.comm",),
    "src.distributed.stream_manager": ("b200fw.dist.streams",),
    "src.distributed.tensor_parallel": ("b200fw.model.qwen3", "b200fw.model.hf_io"),
    "src.distributed.lora": ("b200fw.model.lora",),
    "src.distributed.pipeline_parallel": ("b200fw.pipeline.stages",),
    "src.distributed.pipeline_scheduler": ("b200fw.pipeline.schedule_1f1b",),
    "src.distributed.zero_optim": ("b200fw.optim.zero",),
    "src.distributed.zero_optim_v2": ("b200fw.optim.zero",),
    "src.distributed.zero_optim_v3": ("b200fw.optim.zero",),
    "src.engines.train_engine": ("b200fw.train.engine",),
    "src.engines.c3po_plus": ("b200fw.train.c3po",),
    "src.engines.icepop": ("b200fw.train.icepop",),
    "src.engines.train_worker": ("b200fw.orch.workers",),
    "src.engines.infer_worker": ("b200fw.orch.workers",),
    "src.inference.engine": ("b200fw.infer.engine", "b200fw.infer.config"),
    "src.inference.attention": ("b200fw.infer.attention",),
    "src.inference.context": ("b200fw.infer.context",),
    "src.inference.cuda_graph": ("b200fw.infer.graphs",),
    "src.inference.kv_cache": ("b200fw.infer.kv_cache",),
    "src.inference.model_runner": ("b200fw.infer.runner",),
    "src.inference.prefix_cache": ("b200fw.infer.prefix_cache",),
    "src.inference.radix_cache": ("b200fw.infer.radix_cache",),
    "src.inference.scheduler": ("b200fw.infer.scheduler",),
    "src.inference.speculative": ("b200fw.infer.spec",),
    "src.orchestrator.colocate_orchestrator": ("b200fw.orch.colocate", "b200fw.config"),
    "src.orchestrator.disagg_orchestrator": ("b200fw.orch.disagg",),
    "src.profiling.comm_profiler": ("b200fw.obs.profilers",),
    "src.profiling.compute_profiler": ("b200fw.obs.profilers",),
    "src.profiling.schedule_visualizer": ("b200fw.obs.timeline",),
    "src.reward.gsm8k_reward": ("b200fw.reward.gsm8k",),
    "src.transfer.ipc_transfer": ("b200fw.sync.ipc_transfer", "b200fw.sync.nccl_transfer"),
    "src.transfer.nccl_transfer": ("b200fw.sync.nccl_transfer",),
    "src.transfer.swift_sync": ("b200fw.sync.swift_sync", "b200fw.sync.double_buffer"),
    "src.utils.artifact_writer": ("b200fw.obs.artifacts",),
    "src.utils.eval_utils": ("b200fw.obs.eval_utils",),
    "src.utils.logger": ("b200fw.obs.logging",),
    "src.utils.memory_manager": ("b200fw.obs.memory",),
    "src.utils.memory_profiler": ("b200fw.obs.memory",),
    "src.utils.metrics": ("b200fw.obs.metrics",),
    "src.data.data_pipeline": ("b200fw.data.pipeline",),
    # the packages themselves re-export what their modules define
    "src": (),
    "src.distributed": ("b200fw.dist.context", "b200fw.dist.comm", "b200fw.dist.streams", "b200fw.model.qwen3",
                        "b200fw.model.lora", "b200fw.pipeline.stages", "b200fw.pipeline.schedule_1f1b",
                        "b200fw.optim.zero"),
    "src.engines": ("b200fw.train.engine", "b200fw.train.c3po", "b200fw.train.icepop", "b200fw.orch.workers"),
    "src.inference": ("b200fw.infer",),
    "src.kernels": ("b200fw.ops",),
    "src.orchestrator": ("b200fw.orch", "b200fw.config"),
    "src.profiling": ("b200fw.obs.profilers", "b200fw.obs.timeline"),
    "src.reward": ("b200fw.reward",),
    "src.transfer": ("b200fw.sync",),
    "src.utils": ("b200fw.obs.artifacts", "b200fw.obs.eval_utils", "b200fw.obs.logging", "b200fw.obs.memory",
                  "b200fw.obs.metrics"),
    "src.data": ("b200fw.data",),
}

# names a reference module defines that have no counterpart object here
EXTRA_NAMES: Dict[str, Dict[str, object]] = {
    # src/kernels/__init__.py:8-13 tries to import a Triton flash attention and publishes ``None`` when the module is
    # absent (it is absent from the reference's tree); callers test for ``None`` and use the library path.  Here the
    # attention kernel is native (``b200fw.ops.flash_attention``) and there is no Triton kernel to offer.
    "src.kernels": {"flash_attention_triton": None},
}

_PACKAGES = {name for name in ALIASES if any(other.startswith(name + ".") for other in ALIASES)}


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, targets: Tuple[str, ...]):
        self.targets = targets

    def create_module(self, spec):
        return None                          # the default module object

    def exec_module(self, module: types.ModuleType) -> None:
        sources: List[types.ModuleType] = [importlib.import_module(t) for t in self.targets]
        for src in sources:
            names = getattr(src, "__all__", None) or [n for n in vars(src) if not n.startswith("__")]
            for n in names:
                if n not in module.__dict__ and hasattr(src, n):
                    module.__dict__[n] = getattr(src, n)
        for n, v in EXTRA_NAMES.get(module.__name__, {}).items():
            module.__dict__.setdefault(n, v)
        module.__dict__["__b200fw_targets__"] = self.targets
        if sources and not module.__doc__:
            module.__doc__ = f"Alias of {', '.join(self.targets)} (b200fw.compat)."


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        targets = ALIASES.get(fullname)
        if targets is None:
            return None
        return importlib.machinery.ModuleSpec(fullname, _AliasLoader(targets), is_package=fullname in _PACKAGES)


_finder = _AliasFinder()


def installed() -> bool:
    return _finder in sys.meta_path


def install(force: bool = False) -> bool:
    """Make ``import src...`` resolve to this package.  Returns True when the aliases are active.  A ``src`` package
    that is importable already (the reference itself on ``sys.path``, or any other project's ``src``) is left in place
    and False is returned, unless ``force`` puts the aliases in front of it."""
    if installed():
        return True
    if not force:
        if "src" in sys.modules:
            return False
        try:
            found = importlib.util.find_spec("src")
        except (ImportError, ValueError):
            found = None
        if found is not None:
            return False
    if force:
        for name in [m for m in sys.modules if m == "src" or m.startswith("src.")]:
            del sys.modules[name]
    sys.meta_path.insert(0, _finder)
    return True


def uninstall() -> None:
    """Remove the finder and every alias module it created."""
    if installed():
        sys.meta_path.remove(_finder)
    for name in [m for m, v in sys.modules.items()
                 if (m == "src" or m.startswith("src.")) and isinstance(getattr(v, "__loader__", None), _AliasLoader)]:
        del sys.modules[name]
