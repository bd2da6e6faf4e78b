"""quench6k_b200: a single-GPU, B200-native inference engine for the Recursive Flint MoE decoder."""
__version__ = "0.1.0"

from . import config as config            # noqa: F401  (registers nothing by itself)
from .models import flint as _flint       # noqa: F401  (registers FlintForCausalLM)
from .models import pedotar as _pedotar   # noqa: F401  (registers Pedotar)
from .models import kipedra as _kipedra   # noqa: F401  (registers Kipedra)
from .models import sigusun as _sigusun   # noqa: F401  (registers Sigusun)
from .models import kitodra as _kitodra   # noqa: F401  (registers Kitodra)
from .sampling.params import SamplingParams      # noqa: F401
from .engine.engine import Engine, RequestOutput   # noqa: F401
