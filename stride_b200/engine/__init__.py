from .engine import Engine, EngineBusy, RequestOutput
from .loading import CachePlan, attach_cache, build_model, load_model, plan_cache, random_model, write_random_model
from .runner import ModelRunner
from .trace import TraceError, TraceSession

__all__ = ["Engine", "EngineBusy", "RequestOutput", "CachePlan", "attach_cache", "build_model", "load_model", "plan_cache",
           "random_model", "write_random_model", "ModelRunner", "TraceError", "TraceSession"]
