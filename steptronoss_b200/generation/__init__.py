"""Generation side-car: generatable items, the worker pool that runs them, and the vLLM serving glue."""
from .async_generation import GenerationController, SingleGenerationController  # noqa: F401
from .base_generatable import EndpointGetter, GenableItem, ModelNameGetter, TrainableItem  # noqa: F401
