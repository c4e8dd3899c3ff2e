"""Save/load of pipeline results (Program, Profiles, Plan, SweepResult, MemoryBudgets,
CommunicationInfo, PoolMemoryProfile, TensorChunk), one archive file each."""
from .archive import ArtifactError, archive_kind, load_archive, save_archive
from .objects import (TensorChunk, load_artifact, load_tensor_chunk, save_artifact,
                      save_tensor_chunk)

__all__ = ["ArtifactError", "archive_kind", "load_archive", "save_archive", "TensorChunk",
           "load_artifact", "save_artifact", "load_tensor_chunk", "save_tensor_chunk"]
