from .utils import Placement
from .partitioners.signature import sequential_signatures
