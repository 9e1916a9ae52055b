"""GSPMD-style sharding compiler: capture -> place -> schedule -> Program (+ archive, shares)."""
from .driver import compile_module, compile_program, compiled  # noqa: F401
from .ir import TrainingResult, send, recv  # noqa: F401
from .placement import counts  # noqa: F401
from .runtime import Program  # noqa: F401
from .lower import lower  # noqa: F401,E402
from .fuse import fuse_plan  # noqa: F401,E402
from . import syncmon, check  # noqa: F401,E402
from .bridge import Prepared, prepare, workspace  # noqa: F401,E402
from . import attention_op  # noqa: F401,E402  (registers mesh::attention and its backward)
