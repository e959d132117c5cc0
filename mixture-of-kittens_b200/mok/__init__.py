"""B200-native MoE kernel library with the `mok` interface: `mok.functional` (workspaces, schedules, forward /
backward) over `mok.ops` (the reference's twelve `torch.ops.mok.*` custom ops plus the device router's two) over libmok_b200.so (hand-written sm_100a CUDA)."""
from . import ops
from . import _fake_impls  # noqa: F401  (registers shape functions for torch.compile / FakeTensor)
from . import functional
from .module import MoKMoE, moe_layer, quantize_routed_weights, route

__version__ = "0.1.0"

__all__ = ["__version__", "functional", "ops", "MoKMoE", "moe_layer", "quantize_routed_weights", "route"]
