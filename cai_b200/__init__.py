"""cai_b200: a schedule-driven LLM trainer for B200 GPUs (offline plan compiler, six-stream executor, sm_100a kernels).

The public names are loaded on first use, so ``import cai_b200`` stays cheap and works on a machine without a GPU:

    Engine, synthetic_batch          device executor of a compiled plan (needs a GPU)
    PlanFile, Simulator              plan files and their GPU-free replay under a pricing backend
    pipeline_replay                  all stages of a pipeline replayed together (no closed bubble formula)
    compile_plans, describe          the offline compiler and the decomposition report as a dict
    TokenBatches, lr_at, reshard     data, learning-rate schedule, checkpoint re-layout
"""
__version__ = "0.2.0"

_PUBLIC = {
    "Engine": "cai_b200.runtime.engine", "synthetic_batch": "cai_b200.runtime.engine",
    "PlanFile": "cai_b200.plan", "Simulator": "cai_b200.plan", "compile_plans": "cai_b200.plan", "describe": "cai_b200.plan",
    "PlanError": "cai_b200.plan", "pipeline_replay": "cai_b200.plan",
    "TokenBatches": "cai_b200.utils.data", "lr_at": "cai_b200.utils.schedule", "reshard": "cai_b200.utils.reshard",
}
__all__ = sorted(_PUBLIC) + ["__version__"]


def __getattr__(name):
    import importlib
    if name in _PUBLIC:
        return getattr(importlib.import_module(_PUBLIC[name]), name)
    try:        # plain sub-packages (cai_b200.ops, cai_b200.plan, ...)
        return importlib.import_module(f"{__name__}.{name}")
    except ModuleNotFoundError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
