from dispec_b200.engine.batch import SeqEntry, StepContext
from dispec_b200.engine.llm_engine import LLMEngine
from dispec_b200.engine.runner import ModelRunner
from dispec_b200.engine.scheduler import (ContinuousBatchingEngine, Request, Scheduler, State,
                                          StepPlan)

__all__ = ["SeqEntry", "StepContext", "LLMEngine", "ModelRunner", "ContinuousBatchingEngine",
           "Request", "Scheduler", "State", "StepPlan"]
