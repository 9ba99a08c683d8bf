"""(Reference: atorch/utils/path_utils.py:4-20.)"""
from pathlib import Path
from typing import Optional


def path_is_empty(dir_path: Optional[Path]) -> bool:
    """False only for an existing directory with at least one entry; ``None``, a missing path and a file count as
    empty."""
    if dir_path is None:
        return True
    dir_path = Path(dir_path)
    return not (dir_path.is_dir() and any(True for _ in dir_path.iterdir()))
