from . import functional
from . import module
from . import model
