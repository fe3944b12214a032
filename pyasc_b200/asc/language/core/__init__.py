from .constexpr import ConstExpr, require_constexpr  # noqa: F401
from .dtype import *  # noqa: F401,F403
from .dtype import DataType, KnownTypes  # noqa: F401
from .ir_value import GlobalAddress, PlainValue  # noqa: F401
from .utils import ceildiv  # noqa: F401
