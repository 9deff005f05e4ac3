"""Checkpoint conversion and loading (``.bin`` + ``.json`` shard format)."""
from .converter import ConvertedCheckpoint, convert_dir, convert_shard, validate_dir  # noqa: F401
