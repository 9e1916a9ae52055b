"""Process-level plumbing: context (rank table + symmetric heap), the ``mesh`` c10d backend, verbs."""
from .context import MeshContext, init, context, shutdown  # noqa: F401
