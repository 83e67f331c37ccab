from .spec import LayerRun, ModelSpec

__all__ = ["LayerRun", "ModelSpec"]
