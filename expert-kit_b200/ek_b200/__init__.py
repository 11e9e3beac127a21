"""B200-native expert-worker compute backend for Expert Kit (Python side of the C ABI)."""
from .backend import Backend, BackendConfig, EKError, TileCache  # noqa: F401
from .client import LocalExpertKitClient  # noqa: F401
from . import _lib  # noqa: F401
from .ep import ExpertParallelMoE, BackendStages, plan_exchange, choose_owners  # noqa: F401,E402
from .modules import B200MoEBlock  # noqa: F401,E402
from .vllm import B200GrpcExpert, B200ExpertKitMoE  # noqa: F401,E402
from . import synth  # noqa: F401,E402
