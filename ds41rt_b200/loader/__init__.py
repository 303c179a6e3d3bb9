"""Checkpoint loading: safetensors container validation, the official tensor catalog, shard reads."""
from .safetensors_io import SafetensorsFile, SafetensorsError, write_safetensors  # noqa: F401
from .catalog import Catalog, official_templates, expected_tensors  # noqa: F401
