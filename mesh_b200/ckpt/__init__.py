"""Sharded checkpoints with reshard-on-load, and the sharded AdamW state they carry."""
from .sharded import load_sharded, save_sharded, latest_step  # noqa: F401
