from dispec_b200.engine.batch import SeqEntry, StepContext
from dispec_b200.engine.runner import ModelRunner

__all__ = ["SeqEntry", "StepContext", "ModelRunner"]
