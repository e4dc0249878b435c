"""Built-in architectures; importing this package registers them."""
from dispec_b200.models import qwen2  # noqa: F401
from dispec_b200.models.model import DecoderModel
from dispec_b200.models.spec import LayerCall, ModelSpec

__all__ = ["DecoderModel", "LayerCall", "ModelSpec"]
