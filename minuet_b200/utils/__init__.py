from . import typing
from . import helpers
