"""Parallel-training building blocks: the flat parameter arena and the data-parallel
wrapper (re-exported from `luatorch_b200.distributed`)."""
from .arena import ParamArena, arena_of, storage_units

__all__ = ["ParamArena", "arena_of", "storage_units"]
