from ._C import *  # noqa
from . import _C
