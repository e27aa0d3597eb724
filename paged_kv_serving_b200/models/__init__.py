"""Architectures. Importing this package registers every built-in architecture."""

from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout, collect_param_specs
from paged_kv_serving_b200.models.llama_toy_decoder import LlamaToyDecoder

__all__ = ["LayerCall", "LlamaToyDecoder", "ModelLayout", "collect_param_specs"]
