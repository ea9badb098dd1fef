from . import functional
from . import module
