from . import config  # noqa: F401
from .jit import JITFunction, jit  # noqa: F401
from .launcher import Launcher  # noqa: F401
from .options import CodegenOptions, CompileOptions, LaunchOptions  # noqa: F401
