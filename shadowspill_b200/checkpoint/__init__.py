from .archive import CheckpointError, read_manifest  # noqa: F401
from .load import export_weights, load_checkpoint  # noqa: F401
from .save import save_checkpoint  # noqa: F401
