"""Host runtime: rendezvous, symmetric heap, signal pads, plans."""
from .rendezvous import Rendezvous  # noqa: F401
from .heap import SymmetricHeap, SymmBuffer  # noqa: F401
